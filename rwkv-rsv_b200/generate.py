"""Text-level driver: prompt text -> tokens -> prefill -> GPU self-loop -> text (examples/generate.rs:20-113).

    python -m rwkv_rsv_b200.generate --model model.st --vocab rwkv_vocab_v20230424.json --prompt "The Eiffel tower" --tokens 64

Same flow and defaults as the reference example: the prompt is fed token by token (`infer_tokens`), the self-loop is seeded with
the prompt's last token, sampling uses temperature 0.8, top-k 50, top-p 0.9 and seed 514 unless `--mode argmax`; without a
vocabulary file the default prompt is the token list [304, 25740, 109] and only token ids are printed.
"""
import argparse
import sys
import time

from . import ModelBuilder, SamplerParams
from .tokenizer import Tokenizer

DEFAULT_PROMPT_TOKENS = [304, 25740, 109]  # examples/generate.rs:52


def generate(bundle, prompt_tokens, n, mode="sample", temperature=0.8, top_k=50, top_p=0.9, seed=514):
    """Prefills `prompt_tokens`, then generates `n` tokens on the GPU; returns (generated tokens, seconds of the self-loop)."""
    prompt_tokens = [int(t) for t in prompt_tokens]
    if not prompt_tokens:
        raise ValueError("empty prompt")
    bundle.infer_tokens(prompt_tokens)
    first = prompt_tokens[-1]  # the self-loop's first input is the last prompt token again (examples/generate.rs:56-57)
    t0 = time.perf_counter()
    if mode == "argmax":
        out = bundle.infer_argmax_selfloop(first, n)
    else:
        out = bundle.infer_sample_selfloop(first, n, SamplerParams(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed))
    return [int(t) for t in out], time.perf_counter() - t0


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--vocab", help="vocabulary JSON ({token id: string | [bytes]}); needed for --prompt and for text output")
    ap.add_argument("--prompt", help="prompt text (needs --vocab)")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--mode", choices=["sample", "argmax"], default="sample")
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--seed", type=int, default=514)
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args(argv)
    tok = Tokenizer(open(a.vocab, encoding="utf-8").read()) if a.vocab else None
    if a.prompt is not None and tok is None:
        ap.error("--prompt requires --vocab")  # "PROMPT requires VOCAB_JSON", examples/generate.rs:49
    prompt = tok.encode(a.prompt) if a.prompt is not None else list(DEFAULT_PROMPT_TOKENS)
    bundle = ModelBuilder(a.model, a.device).build()
    out, sec = generate(bundle, prompt, a.tokens, a.mode, a.temperature, a.top_k, a.top_p, a.seed)
    print(f"{a.tokens} tokens in {sec:.3f} s ({a.tokens / max(sec, 1e-9):.1f} tok/s)", file=sys.stderr)
    full = prompt + out
    print(full)
    if tok is not None:
        print(tok.decode(full).decode("utf-8", errors="replace"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
