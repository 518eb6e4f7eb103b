"""``rwkvtune-merge-lora``: fold a LoRA adapter into its base model and write a plain hub directory.

Steps (``rwkvtune/cli/merge_lora.py:112-223``): load the base model, apply and load the adapter,
merge, save ``model.pth`` / ``model.safetensors``; ``config.json`` comes from the base model with
``eos_token_id`` patched from the adapter directory's tokenizer config; tokenizer files are taken
from the adapter directory first; ``merge_info.json`` records provenance.
"""
from __future__ import annotations

import argparse
import json
import shutil
import sys
from pathlib import Path

TOKENIZER_FILES = ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "vocab.txt", "merges.txt",
                   "chat_template.jinja", "generation_config.json")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="rwkvtune-merge-lora", description="Merge LoRA weights into a base RWKV-7 model")
    p.add_argument("--base-model", "-b", required=True, help="base model directory (config.json + weights)")
    p.add_argument("--lora-model", "-l", required=True, help="adapter directory (adapter_config.json + adapter_model.bin)")
    p.add_argument("--output", "-o", required=True, help="output directory for the merged model")
    p.add_argument("--device", default="cpu", choices=["cuda", "cpu"])
    p.add_argument("--precision", default="bf16", choices=["fp32", "fp16", "bf16"])
    p.add_argument("--save-format", default="pth", choices=["pth", "safetensors"])
    return p


def merge(base_model: str, lora_model: str, output: str, device: str = "cpu", precision: str = "bf16",
          save_format: str = "pth") -> str:
    import torch

    from ..models import AutoModel
    from ..peft import load_peft_model

    base, lora, out = Path(base_model), Path(lora_model), Path(output)
    for p, what in ((base, "base model"), (lora, "LoRA model")):
        if not p.is_dir():
            raise FileNotFoundError(f"{what} directory not found: {p}")
    model = AutoModel.from_pretrained(str(base), device=device, dtype=precision)
    model = load_peft_model(model, str(lora))
    model.merge_adapter()
    sd = {k: v.contiguous() for k, v in model.get_merged_state_dict().items()}
    out.mkdir(parents=True, exist_ok=True)
    if save_format == "safetensors":
        from safetensors.torch import save_file

        weights = out / "model.safetensors"
        save_file(sd, str(weights))
    else:
        weights = out / "model.pth"
        torch.save(sd, weights)
    cfg = json.loads((base / "config.json").read_text(encoding="utf-8")) if (base / "config.json").exists() else {}
    tok_cfg_file = lora / "tokenizer_config.json"
    if tok_cfg_file.exists():
        tok_cfg = json.loads(tok_cfg_file.read_text(encoding="utf-8"))
        eos = tok_cfg.get("eos_token")
        for item in tok_cfg.get("additional_special_tokens", []) or []:
            if isinstance(item, dict) and item.get("token") == eos and item.get("id") is not None:
                cfg["eos_token_id"] = item["id"]
                break
    (out / "config.json").write_text(json.dumps(cfg, indent=2, ensure_ascii=False), encoding="utf-8")
    for name in TOKENIZER_FILES:
        src = lora / name if (lora / name).exists() else base / name
        if src.exists():
            shutil.copy(src, out / name)
    info = {"base_model": str(base.resolve()), "lora_model": str(lora.resolve()), "precision": precision,
            "save_format": save_format, "weights_file": weights.name, "merged_by": "rwkvtune-merge-lora"}
    (out / "merge_info.json").write_text(json.dumps(info, indent=2), encoding="utf-8")
    return str(out)


def main(argv=None) -> int:
    a = build_parser().parse_args(sys.argv[1:] if argv is None else argv)
    try:
        out = merge(a.base_model, a.lora_model, a.output, a.device, a.precision, a.save_format)
    except Exception as exc:
        print(f"merge failed: {type(exc).__name__}: {exc}", file=sys.stderr)
        return 1
    print(f"merged model written to {out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
