"""Command line in the manner of the reference's `gguf-infer` (main.rs:61-218).

Kept, with the reference's names, short forms, defaults and meanings:
  --model, -m        model folder (required; must exist)                       main.rs:78-85, :173-177
  --prompt, -p       the prompt; here a list of token ids "1,2,3", repeatable  main.rs:86-93
  --max-tokens, -n   tokens to generate (default 512)                          main.rs:65, :94-101
  --temperature, -t  sampling temperature, 0 = greedy (default 0.8)            main.rs:66
  --top-k, -k        top-k (default 40)                                        main.rs:67
  --top-p            nucleus (default 0.95)                                    main.rs:68
  --seed, -s         sampler seed (default 12345)                              main.rs:69
  --max-seq-len      override the model's context length                      main.rs:134-142
  --help, -h         usage, exit 0; an unknown argument prints usage, exit 1  main.rs:160-168
The repetition penalty is 1.1 over 64 tokens as the reference hard-wires it (main.rs:187-188);
--repetition-penalty 1 switches it off.  --cpu / --gpu are replaced by --dtype (which numeric
path); --interactive and --system belong to the text front-end, which this library does not have.
"""
from __future__ import annotations

import os
import sys
import time

USAGE = """B200 dense-decoder inference (token ids in, token ids out)

Usage: gguf-infer --model <folder> --prompt "<id,id,...>" [options]

Options:
  --model, -m        Path to the model folder: config.json + model.safetensors (required)
  --prompt, -p       Prompt as comma- or space-separated token ids; repeat for a batch
  --prompt-file      File with one prompt (token ids) per line
  --max-tokens, -n   Maximum tokens to generate (default: 512)
  --temperature, -t  Sampling temperature, 0 = greedy (default: 0.8)
  --top-k, -k        Top-K sampling, 0 = off (default: 40)
  --top-p            Top-P nucleus sampling, 1 = off (default: 0.95)
  --repetition-penalty  Repetition penalty over the last 64 tokens, 1 = off (default: 1.1)
  --seed, -s         Random seed (default: 12345)
  --max-seq-len      Override max sequence length
  --stop-ids         Stop token ids (default: the model's eos ids)
  --dtype            bfloat16 (default) or float32
  --help, -h         Show this help message
"""


class CliError(Exception):
    pass


def _ids(text: str) -> list:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise CliError(f"Invalid token id list: {text!r}") from None


def parse_args(argv: list) -> dict:
    """Hand-rolled like the reference's parser (main.rs:61-196).  Returns a dict, or raises
    CliError; 'help' is set when usage was asked for."""
    a = {"model": None, "prompts": [], "max_tokens": 512, "temperature": 0.8, "top_k": 40, "top_p": 0.95,
         "repetition_penalty": 1.1, "seed": 12345, "max_seq_len": None, "stop_ids": None,
         "dtype": "bfloat16", "help": False}
    i = 0

    def value(flag):
        nonlocal i
        i += 1
        if i >= len(argv):
            raise CliError(f"{flag} requires a value")
        return argv[i]

    def number(flag, kind):
        v = value(flag)
        try:
            return kind(v)
        except ValueError:
            raise CliError(f"Invalid {flag}: {v!r}") from None

    while i < len(argv):
        arg = argv[i]
        if arg in ("--model", "-m"):
            a["model"] = value("--model")
        elif arg in ("--prompt", "-p"):
            a["prompts"].append(_ids(value("--prompt")))
        elif arg == "--prompt-file":
            path = value("--prompt-file")
            try:
                with open(path) as f:
                    a["prompts"].extend(_ids(line) for line in f if line.strip())
            except OSError as e:
                raise CliError(f"Cannot read {path}: {e.strerror}") from None
        elif arg in ("--max-tokens", "-n"):
            a["max_tokens"] = number("--max-tokens", int)
        elif arg in ("--temperature", "-t"):
            a["temperature"] = number("--temperature", float)
        elif arg in ("--top-k", "-k"):
            a["top_k"] = number("--top-k", int)
        elif arg == "--top-p":
            a["top_p"] = number("--top-p", float)
        elif arg == "--repetition-penalty":
            a["repetition_penalty"] = number("--repetition-penalty", float)
        elif arg in ("--seed", "-s"):
            a["seed"] = number("--seed", int)
        elif arg == "--max-seq-len":
            a["max_seq_len"] = number("--max-seq-len", int)
        elif arg == "--stop-ids":
            a["stop_ids"] = _ids(value("--stop-ids"))
        elif arg == "--dtype":
            a["dtype"] = value("--dtype")
            if a["dtype"] not in ("bfloat16", "float32", "bf16", "fp32"):
                raise CliError(f"Invalid --dtype: {a['dtype']!r}")
        elif arg in ("--help", "-h"):
            a["help"] = True
            return a
        elif arg in ("--interactive", "-i", "--system", "--cpu", "--gpu"):
            raise CliError(f"{arg} is not available: this engine takes token ids and runs on the GPU only")
        else:
            raise CliError(f"Unknown argument: {arg}")
        i += 1
    if a["model"] is None:
        raise CliError("--model is required")
    if not os.path.exists(a["model"]):
        raise CliError(f"Model file not found: {a['model']}")
    if not a["prompts"]:
        raise CliError("--prompt is required")
    if any(len(p) == 0 for p in a["prompts"]):
        raise CliError("a prompt has no token ids")
    return a


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        a = parse_args(argv)
    except CliError as e:
        print(f"Error: {e}", file=sys.stderr)
        print(USAGE, file=sys.stderr)
        return 1
    if a["help"]:
        print(USAGE, file=sys.stderr)
        return 0

    from .api import Model
    from .sampling.params import SamplerConfig
    try:
        model = Model.load(a["model"], a["max_seq_len"], dtype=a["dtype"])
    except Exception as e:                          # main.rs:257-263
        print(f"Failed to load model: {e}", file=sys.stderr)
        return 1
    cfg = SamplerConfig(temperature=a["temperature"], top_k=a["top_k"], top_p=a["top_p"],
                        repetition_penalty=a["repetition_penalty"], repetition_window=64, seed=a["seed"])
    t0 = time.time()
    results = model.generate(a["prompts"], a["max_tokens"], cfg, stop_ids=a["stop_ids"])
    dt = time.time() - t0
    for r in results:
        print(" ".join(str(t) for t in r.tokens))
    n = sum(len(r.tokens) for r in results)
    print(f"{n} tokens in {dt:.3f} s ({n / dt:.1f} tok/s), finish: "
          + ", ".join(r.finish_reason for r in results), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
