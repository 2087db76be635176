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
Added for a library that takes token ids and may run without a checkpoint:
  --random-config FILE + --weights-seed S   a config.json alone: weights N(0, 0.02) from the seed, on the device
  --random-prompts B:MIN:MAX                B prompts of seeded random ids, lengths uniform in MIN..MAX
  --slots N                                 sequences that may be live at once (larger batches run in waves)
  --print-logits-topk K                     the K largest logits after each prompt, before generating
  --bench                                   after generating, one JSON line on standard error: steps, prompt and
                                            generated tokens, seconds, tokens per second, bytes copied, the model's
                                            bytes on the device
  --dump-layer-stats                        min / max / mean / first values of the hidden vector at position 0
                                            after every layer, as debug builds of the reference print them
                                            (transformer.rs:80-96)
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
  --model, -m        Path to the model folder: config.json + model.safetensors (required unless --random-config)
  --random-config    A config.json alone: run it with random weights (see --weights-seed)
  --weights-seed     Seed of the random weights (default: 0)
  --prompt, -p       Prompt as comma- or space-separated token ids; repeat for a batch
  --prompt-file      File with one prompt (token ids) per line
  --random-prompts   B:MIN:MAX, B prompts of random ids with lengths in MIN..MAX (seeded by --seed)
  --max-tokens, -n   Maximum tokens to generate (default: 512)
  --temperature, -t  Sampling temperature, 0 = greedy (default: 0.8)
  --top-k, -k        Top-K sampling, 0 = off (default: 40)
  --top-p            Top-P nucleus sampling, 1 = off (default: 0.95)
  --repetition-penalty  Repetition penalty over the last 64 tokens, 1 = off (default: 1.1)
  --seed, -s         Random seed (default: 12345)
  --max-seq-len      Override max sequence length
  --stop-ids         Stop token ids (default: the model's eos ids)
  --dtype            bfloat16 (default) or float32
  --slots            Sequences live at once (default: as many as the cache holds)
  --print-logits-topk  Print the K largest logits after each prompt
  --dump-layer-stats Print per-layer statistics of the hidden state at position 0
  --bench            Print the run's counts, rates and the model's memory as one JSON line
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
         "dtype": "bfloat16", "help": False, "random_config": None, "weights_seed": 0, "random_prompts": None,
         "slots": None, "logits_topk": 0, "layer_stats": False, "bench": False}
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
        elif arg == "--random-config":
            a["random_config"] = value("--random-config")
        elif arg == "--weights-seed":
            a["weights_seed"] = number("--weights-seed", int)
        elif arg == "--random-prompts":
            text = value("--random-prompts")
            try:
                b, lo, hi = (int(x) for x in text.split(":"))
            except ValueError:
                raise CliError(f"Invalid --random-prompts: {text!r} (want B:MIN:MAX)") from None
            if b < 1 or lo < 1 or hi < lo:
                raise CliError(f"Invalid --random-prompts: {text!r} (want B >= 1 and 1 <= MIN <= MAX)")
            a["random_prompts"] = (b, lo, hi)
        elif arg == "--slots":
            a["slots"] = number("--slots", int)
            if a["slots"] < 1:
                raise CliError("Invalid --slots: at least 1")
        elif arg == "--print-logits-topk":
            a["logits_topk"] = number("--print-logits-topk", int)
        elif arg == "--dump-layer-stats":
            a["layer_stats"] = True
        elif arg == "--bench":
            a["bench"] = True
        elif arg in ("--help", "-h"):
            a["help"] = True
            return a
        elif arg in ("--interactive", "-i", "--system", "--cpu", "--gpu"):
            raise CliError(f"{arg} is not available: this engine takes token ids and runs on the GPU only")
        else:
            raise CliError(f"Unknown argument: {arg}")
        i += 1
    if a["model"] is None and a["random_config"] is None:
        raise CliError("--model is required")
    if a["model"] is not None and a["random_config"] is not None:
        raise CliError("--model and --random-config exclude each other")
    path = a["model"] if a["model"] is not None else a["random_config"]
    if not os.path.exists(path):
        raise CliError(f"Model file not found: {path}")
    if not a["prompts"] and a["random_prompts"] is None:
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
        if a["random_config"] is not None:
            import json
            from .config.registry import config_from_dict
            with open(a["random_config"], encoding="utf-8") as f:
                config = config_from_dict(json.load(f))
            model = Model.random(config, seed=a["weights_seed"], dtype=a["dtype"], max_seq_len=a["max_seq_len"],
                                 n_slots=a["slots"])
        else:
            model = Model.load(a["model"], a["max_seq_len"], dtype=a["dtype"], n_slots=a["slots"])
    except Exception as e:                          # main.rs:257-263
        print(f"Failed to load model: {e}", file=sys.stderr)
        return 1
    prompts = list(a["prompts"])
    vocab = model.engine.model.spec.vocab_size
    if a["random_prompts"] is not None:
        import random
        b, lo, hi = a["random_prompts"]
        rng = random.Random(a["seed"])
        prompts += [[rng.randrange(vocab) for _ in range(rng.randint(lo, hi))] for _ in range(b)]
    if a["logits_topk"] > 0 or a["layer_stats"]:
        from .engine.model import LayerProbe
        for i, p in enumerate(prompts):
            stats = [] if a["layer_stats"] else None
            row = model.logits(p, "last", layer_stats=stats)[0]
            if stats is not None:
                print(f"prompt {i}: hidden state at position 0", file=sys.stderr)
                for label, st in stats:
                    print(LayerProbe.format(label, st), file=sys.stderr)
            if a["logits_topk"] > 0:
                top = row.topk(min(a["logits_topk"], vocab))
                print(f"prompt {i}: top logits " + " ".join(f"{int(t)}:{float(v):.4f}" for v, t in
                                                             zip(top.values.tolist(), top.indices.tolist())),
                      file=sys.stderr)
    cfg = SamplerConfig(temperature=a["temperature"], top_k=a["top_k"], top_p=a["top_p"],
                        repetition_penalty=a["repetition_penalty"], repetition_window=64, seed=a["seed"])
    t0 = time.time()
    results = model.generate(prompts, a["max_tokens"], cfg, stop_ids=a["stop_ids"], max_batch=a["slots"])
    dt = time.time() - t0
    for r in results:
        print(" ".join(str(t) for t in r.tokens))
    n = sum(len(r.tokens) for r in results)
    print(f"{n} tokens in {dt:.3f} s ({n / dt:.1f} tok/s), finish: "
          + ", ".join(r.finish_reason for r in results), file=sys.stderr)
    if a["bench"]:
        import json
        stats = {k: v for k, v in model.last_stats.items() if k != "step_times"}
        print(json.dumps({**stats, **model.memory()}), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
