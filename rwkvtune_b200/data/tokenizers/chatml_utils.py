"""ChatML set-up and checks for a tokenizer (``rwkvtune/data/tokenizers/chatml_utils.py:27-347``)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

CHATML_TEMPLATE = ("{% for message in messages %}{{ '<|im_start|>' + message['role'] + '\n' + message['content'] + "
                   "'<|im_end|>' + '\n' }}{% endfor %}{% if add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}")
IM_START, IM_END = "<|im_start|>", "<|im_end|>"


class ChatMLConfigError(Exception):
    pass


class ChatMLValidationError(Exception):
    pass


def validate_chatml_tokenizer(tokenizer) -> Tuple[bool, List[str]]:
    errors: List[str] = []
    template = getattr(tokenizer, "chat_template", None)
    if template is None:
        return False, ["tokenizer.chat_template is not set"]
    for marker in (IM_START, IM_END):
        if marker not in template:
            errors.append(f"chat_template does not contain the ChatML marker {marker}")
    added = getattr(tokenizer, "additional_special_tokens", {})
    for marker in (IM_START, IM_END):
        if marker not in added:
            errors.append(f"{marker} is not registered as a special token")
        elif len(tokenizer.encode(marker, add_special_tokens=False)) != 1:
            errors.append(f"{marker} does not encode to a single id")
    if getattr(tokenizer, "eos_token", None) != IM_END:
        errors.append(f"eos_token is {getattr(tokenizer, 'eos_token', None)!r}, expected {IM_END!r}")
    return not errors, errors


def setup_chatml_tokenizer(tokenizer, chat_template_path: Optional[str] = None, verify: bool = True,
                           raise_on_error: bool = True, im_end_id: Optional[int] = 0) -> Dict[str, Any]:
    """Register ``<|im_start|>`` / ``<|im_end|>``, make ``<|im_end|>`` the EOS (by default re-mapped to the
    unused id 0 so the embedding matrix does not grow) and install a ChatML template."""
    results: Dict[str, Any] = {"success": False, "added_tokens": 0, "template_set": False, "warnings": [], "errors": []}
    try:
        results["added_tokens"] += tokenizer.add_special_tokens({"additional_special_tokens": [IM_START]})
        if im_end_id is not None:
            tokenizer.add_special_token_with_id(IM_END, im_end_id, set_as="eos_token")
            tokenizer.pad_token, tokenizer.pad_token_id = IM_END, im_end_id
        else:
            results["added_tokens"] += tokenizer.add_special_tokens({"additional_special_tokens": [IM_END],
                                                                     "eos_token": IM_END, "pad_token": IM_END})
        if chat_template_path:
            with open(chat_template_path, "r", encoding="utf-8") as fh:
                tokenizer.chat_template = fh.read()
        else:
            tokenizer.chat_template = CHATML_TEMPLATE
        results["template_set"] = True
        if verify:
            ok, errs = validate_chatml_tokenizer(tokenizer)
            results["errors"].extend(errs)
            ok2, diag = verify_chatml_formatting(tokenizer)
            results["errors"].extend(diag.get("errors", []))
            results["success"] = ok and ok2
        else:
            results["success"] = True
    except Exception as exc:  # configuration problems are reported, not hidden
        results["errors"].append(f"{type(exc).__name__}: {exc}")
    if not results["success"] and raise_on_error:
        raise ChatMLConfigError("; ".join(results["errors"]) or "ChatML set-up failed")
    return results


def verify_chatml_formatting(tokenizer, test_messages: Optional[List[Dict[str, str]]] = None,
                             raise_on_error: bool = False) -> Tuple[bool, Dict[str, Any]]:
    msgs = test_messages or [{"role": "system", "content": "You are helpful."}, {"role": "user", "content": "Hi"},
                             {"role": "assistant", "content": "Hello!"}]
    diag: Dict[str, Any] = {"errors": []}
    try:
        text = tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=False)
        ids = tokenizer.encode(text, add_special_tokens=False)
        diag.update(text=text, num_tokens=len(ids))
        start_id = tokenizer.additional_special_tokens.get(IM_START)
        end_id = tokenizer.additional_special_tokens.get(IM_END)
        if ids.count(start_id) != len(msgs) or ids.count(end_id) != len(msgs):
            diag["errors"].append("special-token counts do not match the number of messages")
        if tokenizer.decode(ids) != text:
            diag["errors"].append("encode/decode round trip changed the text")
    except Exception as exc:
        diag["errors"].append(f"{type(exc).__name__}: {exc}")
    ok = not diag["errors"]
    if not ok and raise_on_error:
        raise ChatMLValidationError("; ".join(diag["errors"]))
    return ok, diag


def print_chatml_diagnostics(tokenizer, verbose: bool = True) -> None:
    ok, errs = validate_chatml_tokenizer(tokenizer)
    print(f"ChatML configuration: {'OK' if ok else 'INVALID'}")
    for e in errs:
        print(f"  - {e}")
    if verbose:
        print(f"  eos_token={tokenizer.eos_token!r} (id {tokenizer.eos_token_id}), vocab_size={tokenizer.vocab_size}")
        print(f"  special tokens: {getattr(tokenizer, 'additional_special_tokens', {})}")
