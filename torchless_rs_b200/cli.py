"""Command line in the manner of the reference's `torchless [OPTIONS] <model_path> [prompt]`
(src/main.rs:28-91, parsing :179-345): the same option names and meanings where this
library has the feature, a hand-rolled parser, an unknown option is an error with exit
code 1 (:335-339).  The prompt is a list of token ids, since the tokenizer is outside
this library; several prompts separated by ';' form a batch of unequal lengths.

Options of the reference that stand for features outside this library (--lazy,
--speculative, --chat, --system, --show-thinking, --socket, --chat-save-root,
--list-backends, --kv-dtype) are refused by name, with the reason.
"""
from __future__ import annotations

import sys
from typing import List, Optional

USAGE = """Usage: {prog} [OPTIONS] <model_path> [prompt-token-ids]

Options:
  --max-tokens <N>      Maximum tokens to generate per response
                        (default: max-seq-len/4, clamped to 1024..32768)
  --max-seq-len <N>     Maximum sequence length / context window
                        (default: model's max_position_embeddings)
  --temperature <T>     Sampling temperature (default: 0.7)
                        0.0 = greedy/deterministic, 0.7 = balanced, 1.0+ = creative
  --top-k <K>           Top-k sampling: only consider the top K tokens
  --top-p <P>           Nucleus sampling: keep smallest set of tokens with
                        cumulative probability >= P
  --backend <BACKEND>   Compute backend: auto or cuda (the only one here)
  --dtype <TYPE>        bfloat16 (default) or float32 (true 32-bit everywhere)
  --seed <S>            Seed of the sampling draws (default: 0)
  --random-weights      Draw the weights from --weights-seed instead of reading
                        model.safetensors (<model_path> then needs config.json only)
  --weights-seed <S>    Seed of --random-weights (default: 0)
  --save-weights        With --random-weights: also write model.safetensors into
                        <model_path> (the same values)
  --stop <IDS>          Comma-separated stop token ids (default: none, as the
                        reference's single-shot mode; 'config' = the model's end tokens)
  --debug               Enable debug output
  --help                Show this help message

<model_path> is a folder with config.json and model.safetensors.
[prompt-token-ids] are integers separated by spaces or commas; ';' separates the
prompts of a batch.  Output: the generated token ids, one line per prompt.

Examples:
  {prog} model_dir "1 415 3211 302"
  {prog} --temperature 0 --max-tokens 32 model_dir "1,5,9 ; 1,7"
"""

_OUTSIDE = {
    "--lazy": "weights live in device memory; there is no on-demand loading mode",
    "--speculative": "speculative decoding is outside this library",
    "--chat": "chat mode is outside this library",
    "--system": "chat mode is outside this library",
    "--show-thinking": "chat mode is outside this library",
    "--socket": "servers are outside this library",
    "--chat-save-root": "servers are outside this library",
    "--list-backends": "there is one backend, CUDA on sm_100a",
    "--kv-dtype": "the cache has the type of --dtype",
}


def resolve_max_tokens(user_value: Optional[int], max_seq_len: int) -> int:
    """Default max_seq_len / 4, clamped to 2048..32768 for contexts of 4096 or more
    and to 1024..32768 below (src/main.rs:144-153)."""
    if user_value is not None:
        return user_value
    lo = 2048 if max_seq_len >= 4096 else 1024
    return min(max(max_seq_len // 4, lo), 32768)


def parse_prompts(text: str, vocab: Optional[int] = None) -> List[List[int]]:
    prompts = []
    for part in text.split(";"):
        ids = part.replace(",", " ").split()
        if not ids:
            continue
        try:
            toks = [int(t) for t in ids]
        except ValueError as e:
            raise ValueError(f"the prompt must be token ids (integers): {e}") from None
        prompts.append(toks)
    return prompts


class CliError(Exception):
    pass


def parse_args(argv: List[str]) -> dict:
    opts = dict(max_tokens=None, max_seq_len=None, temperature=0.7, top_k=None, top_p=None,
                dtype="bfloat16", seed=0, stop=(), debug=False, help=False, positional=[],
                random_weights=False, weights_seed=0, save_weights=False)
    i = 0

    def value(name: str, conv):
        nonlocal i
        if i + 1 >= len(argv):
            raise CliError(f"Error: {name} requires a value")
        i += 1
        try:
            return conv(argv[i])
        except ValueError:
            raise CliError(f"Error: invalid value '{argv[i]}' for {name}") from None

    while i < len(argv):
        a = argv[i]
        if a in ("--help", "-h"):
            opts["help"] = True
        elif a == "--max-tokens":
            opts["max_tokens"] = value(a, int)
        elif a == "--max-seq-len":
            opts["max_seq_len"] = value(a, int)
        elif a == "--temperature":
            opts["temperature"] = value(a, float)
        elif a == "--top-k":
            opts["top_k"] = value(a, int)
        elif a == "--top-p":
            opts["top_p"] = value(a, float)
        elif a == "--dtype":
            opts["dtype"] = value(a, str)
        elif a == "--seed":
            opts["seed"] = value(a, int)
        elif a == "--random-weights":
            opts["random_weights"] = True
        elif a == "--weights-seed":
            opts["weights_seed"] = value(a, int)
        elif a == "--save-weights":
            opts["save_weights"] = True
        elif a == "--stop":
            v = value(a, str)
            opts["stop"] = "config" if v == "config" else tuple(int(t) for t in v.split(",") if t)
        elif a == "--backend":
            b = value(a, str)
            if b not in ("auto", "cuda"):
                raise CliError(f"Error: backend '{b}' is not available; this library runs on CUDA only")
        elif a == "--debug":
            opts["debug"] = True
        elif a in _OUTSIDE:
            raise CliError(f"Error: option '{a}' is not available: {_OUTSIDE[a]}")
        elif a.startswith("-") and not a.lstrip("-").replace(",", "").replace(" ", "").isdigit():
            raise CliError(f"Error: unknown option '{a}'\nUse --help for usage information.")
        else:
            opts["positional"].append(a)
        i += 1
    return opts


def main(argv: Optional[List[str]] = None, prog: str = "torchless") -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        opts = parse_args(argv)
    except CliError as e:
        print(e, file=sys.stderr)
        return 1
    if opts["help"]:
        print(USAGE.format(prog=prog), file=sys.stderr)
        return 0
    pos = opts["positional"]
    if not pos:
        print(USAGE.format(prog=prog), file=sys.stderr)
        return 1
    model_dir = pos[0]
    try:
        prompts = parse_prompts(" ".join(pos[1:])) if len(pos) > 1 else []
    except ValueError as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1

    from . import api
    from .config import load_config
    try:
        config = load_config(model_dir)
    except Exception as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    max_seq_len = opts["max_seq_len"] or config.max_position_embeddings
    if opts["max_seq_len"] and opts["max_seq_len"] > config.max_position_embeddings:
        print(f"WARNING: --max-seq-len {max_seq_len} exceeds the model's trained context length "
              f"({config.max_position_embeddings}).", file=sys.stderr)
    max_tokens = resolve_max_tokens(opts["max_tokens"], max_seq_len)
    if not prompts:
        bos = config.bos_token_id if config.bos_token_id is not None else 1
        prompts = [[bos]]
    longest = max(len(p) for p in prompts)
    if longest >= max_seq_len:
        print(f"Error: a prompt of {longest} tokens does not fit --max-seq-len {max_seq_len}",
              file=sys.stderr)
        return 1
    max_tokens = min(max_tokens, max_seq_len - longest + 1)
    per_seq = (min(max_seq_len, longest + max_tokens) + 63) // 64 * 64
    if opts["debug"]:
        print(f"Loading {model_dir} ({opts['dtype']}), {len(prompts)} prompt(s), "
              f"max_tokens {max_tokens}, max_seq_len {max_seq_len}", file=sys.stderr)
    if opts["save_weights"] and not opts["random_weights"]:
        print("Error: --save-weights goes with --random-weights", file=sys.stderr)
        return 1
    try:
        if opts["random_weights"]:
            if opts["save_weights"]:
                from .weights import write_random_model
                write_random_model(config, model_dir, opts["weights_seed"], api.parse_dtype(opts["dtype"]),
                                   "cuda:0")
            model = api.from_random(config, seed=opts["weights_seed"], dtype=opts["dtype"],
                                    max_tokens=per_seq * len(prompts), max_batch=len(prompts),
                                    max_seq_len=max_seq_len)
        else:
            model = api.load(model_dir, dtype=opts["dtype"], max_tokens=per_seq * len(prompts),
                             max_batch=len(prompts), max_seq_len=max_seq_len)
    except Exception as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    stop = config.eos_token_ids if opts["stop"] == "config" else opts["stop"]
    single = len(prompts) == 1

    def on_token(i: int, tok: int) -> None:
        if single:
            sys.stdout.write(f"{tok} ")
            sys.stdout.flush()

    results = model.generate(prompts, max_tokens=max_tokens, temperature=opts["temperature"],
                             top_k=opts["top_k"], top_p=opts["top_p"], stop_ids=stop,
                             seed=opts["seed"], on_token=on_token)
    if single:
        sys.stdout.write("\n")
    else:
        for r in results:
            print(" ".join(str(t) for t in r.tokens))
    if opts["debug"]:
        for i, r in enumerate(results):
            print(f"prompt {i}: {r.prompt_len} tokens in, {len(r.tokens)} out, "
                  f"stopped_at_eos={r.stopped_at_eos}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
