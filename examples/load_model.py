"""Prepare the model directory of the end-to-end run.

    python examples/load_model.py [--out Llama-3.2-1B] [--tiny] [--dtype bfloat16] [--download meta-llama/Llama-3.2-1B]

The counterpart of the reference's motivation/load_model.py, which downloads a Llama checkpoint and its tokenizer
and saves both locally.  With ``--download NAME`` (needs ``transformers`` and network access) this does the same;
otherwise it writes a random-init checkpoint of the Llama-3.2-1B shape (``--tiny``: a 2-layer toy) in the Hugging
Face layout (``config.json`` + ``model.safetensors``), which ``examples/train_ddp.py --model-dir`` and
``transformers.AutoModelForCausalLM.from_pretrained`` both load.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from stragglar_b200.models import LlamaConfig, LlamaForCausalLM  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="Llama-3.2-1B")
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--download", default=None, metavar="NAME", help="Hugging Face model name to fetch instead")
    args = ap.parse_args()
    if args.download:
        try:
            from transformers import AutoModelForCausalLM, AutoTokenizer
            AutoTokenizer.from_pretrained(args.download).save_pretrained(args.out)
            AutoModelForCausalLM.from_pretrained(args.download).save_pretrained(args.out)
            print(f"model and tokenizer of {args.download} saved to {args.out}")
            return 0
        except Exception as e:
            print(f"download failed ({type(e).__name__}: {e}); writing a random-init checkpoint instead", file=sys.stderr)
    torch.manual_seed(args.seed)
    cfg = LlamaConfig.tiny() if args.tiny else LlamaConfig.llama32_1b()
    model = LlamaForCausalLM(cfg).to(getattr(torch, args.dtype))
    model.save_pretrained(args.out)
    print(f"random-init model ({cfg.num_parameters() / 1e9:.3f} B parameters, {args.dtype}) saved to {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
