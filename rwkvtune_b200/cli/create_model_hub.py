"""``rwkvtune-create-hub``: command-line front end of :func:`create_model_hub`
(flags as in ``rwkvtune/cli/create_model_hub.py:61-162``)."""
from __future__ import annotations

import argparse
import sys


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="rwkvtune-create-hub", description="Create a standard RWKV-7 model directory")
    p.add_argument("--output-dir", "-o", required=True)
    p.add_argument("--model-file", "-m", default=None)
    p.add_argument("--config-name", "-c", default=None, help='preset such as "rwkv7-0.1b" or "1.5b"')
    p.add_argument("--vocab-file", default=None)
    p.add_argument("--chat-template", default=None)
    p.add_argument("--model-name", default=None)
    p.add_argument("--description", default=None)
    for name in ("n-layer", "n-embd", "vocab-size", "head-size-a", "ctx-len", "dim-att-lora", "dim-gate-lora", "dim-mv-lora"):
        p.add_argument(f"--{name}", type=int, default=None)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-p", type=float, default=0.85)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--max-length", type=int, default=1024)
    p.add_argument("--eos-token", default="\n\n")
    p.add_argument("--model-max-length", type=int, default=4096)
    p.add_argument("--copy-weights", action="store_true", default=True, help="copy the weight file (default)")
    p.add_argument("--link-weights", "--no-copy", dest="link_weights", action="store_true",
                   help="symlink the weight file instead of copying it")
    p.add_argument("--verbose", action="store_true", help="print the resolved settings and full tracebacks")
    p.add_argument("--save-format", choices=["pth", "safetensors"], default="pth")
    p.add_argument("--overwrite", action="store_true")
    p.add_argument("--list-configs", action="store_true")
    return p


def main(argv=None) -> int:
    if argv is None:
        argv = sys.argv[1:]
    if "--list-configs" in argv:
        from ..configs import list_available_models

        for name in list_available_models():
            print(name)
        return 0
    a = build_parser().parse_args(argv)
    from ..utils import create_model_hub

    if a.verbose:
        for key, value in sorted(vars(a).items()):
            print(f"  {key}: {value}")
    try:
        out = _create(a, create_model_hub)
    except Exception as err:      # the reference reports the error and exits 1 (cli/create_model_hub.py:255-261)
        print(f"error: {err}", file=sys.stderr)
        if a.verbose:
            import traceback

            traceback.print_exc()
        return 1
    print(f"model directory written to {out}")
    return 0


def _create(a, create_model_hub):
    return create_model_hub(
        output_dir=a.output_dir, model_file=a.model_file, config_name=a.config_name, vocab_file=a.vocab_file,
        chat_template_file=a.chat_template, model_name=a.model_name, description=a.description, n_layer=a.n_layer,
        n_embd=a.n_embd, vocab_size=a.vocab_size, head_size_a=a.head_size_a, ctx_len=a.ctx_len,
        dim_att_lora=a.dim_att_lora, dim_gate_lora=a.dim_gate_lora, dim_mv_lora=a.dim_mv_lora,
        temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, repetition_penalty=a.repetition_penalty,
        max_length=a.max_length, eos_token=a.eos_token, model_max_length=a.model_max_length,
        copy_weights=not a.link_weights, save_format=a.save_format, overwrite=a.overwrite)


if __name__ == "__main__":
    raise SystemExit(main())
