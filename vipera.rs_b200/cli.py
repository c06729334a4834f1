"""Command line in the reference's manner: ``vipera <command> <model> [flags]``.

Commands and flags follow bins/vipera/src/main.rs:32-64 and the contract in
specs/001-vipera-rs-engine/contracts/cli.md: ``generate`` (main.rs:548-756: --prompt,
--max-tokens 32, --ctx, --temperature 0, --top-k 40, --top-p 0.95, --min-p 0.05,
--repetition-penalty 1.0, --seed 0, --json), ``model-info`` (main.rs:161-184) and ``plan``
(main.rs:186-251, exit code 3 when the plan is infeasible).  Flags are parsed by hand as
there; an unknown flag is a usage error (exit code 1).  Exit codes: 0 ok, 1 usage, 2 bad
input, 3 infeasible, 4 internal (crates/vipera-errors/src/lib.rs:94-104).

Differences that come with this engine's scope: the tokenizer is not part of it, so
``--prompt`` takes token ids ("151 2040 17") and tokens are printed as ids; ``--dtype``
chooses bfloat16 or float32; ``random-weights`` writes a model folder from a config.json
and a seed.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import List, Optional

from .errors import InfeasibleError, InternalError, InvalidArgumentError, UsageError, ViperaError

USAGE = """usage: vipera <command> [arguments]

commands:
  generate <model> --prompt "IDS" [--max-tokens N] [--ctx N] [--temperature T] [--top-k K]
           [--top-p P] [--min-p P] [--repetition-penalty F] [--presence-penalty F]
           [--frequency-penalty F] [--seed S] [--dtype bfloat16|float32] [--page-size N] [--json]
  model-info <model> [--json]
  plan <model> [--ctx N] [--batch N] [--dtype bfloat16|float32] [--device-bytes N] [--page-size N] [--json]
  random-weights <config.json> <out-dir> [--seed S] [--dtype bfloat16|float32]

exit codes: 0 ok, 1 usage, 2 bad input, 3 infeasible, 4 internal
"""


def _value(args: List[str], index: int, flag: str) -> str:
    if index + 1 >= len(args):
        raise UsageError(f"{flag} needs a value")
    return args[index + 1]


def _number(flag: str, text: str, kind=int):
    try:
        return kind(text)
    except ValueError:
        raise InvalidArgumentError(f"{flag} needs a number, got {text!r}") from None


def _parse(args: List[str], command: str, valued: dict, switches: set, positional: int):
    """Hand parsing: ``valued`` maps a flag to (name, converter)."""
    found, places = {}, []
    index = 0
    while index < len(args):
        arg = args[index]
        if arg in switches:
            found[arg.lstrip("-").replace("-", "_")] = True
        elif arg in valued:
            name, kind = valued[arg]
            text = _value(args, index, arg)
            found[name] = text if kind is str else _number(arg, text, kind)
            index += 1
        elif arg.startswith("-") and not arg.lstrip("-").replace(".", "").isdigit():
            raise UsageError(f'unknown flag "{arg}" for {command}')
        else:
            if len(places) >= positional:
                raise UsageError(f'unexpected extra argument "{arg}"')
            places.append(arg)
        index += 1
    return found, places


def _model_report(model_dir: str) -> dict:
    """What the folder holds, by the architecture-neutral description and the file itself
    (bins/vipera/src/main.rs:161-184)."""
    from .config import load_config
    from .engine import planner
    from .parts import model_schema
    from .weights import SafetensorsSource, check_source

    arch, config = load_config(model_dir)
    spec = arch.model_spec(config)
    source = SafetensorsSource(model_dir)
    schema = model_schema(spec)
    check_source(schema, source)
    dtypes, total_bytes, parameters = {}, 0, 0
    for name in source.names():
        count = 1
        for extent in source.shape(name):
            count *= extent
        dtype = str(source.stored_dtype(name)).replace("torch.", "")
        dtypes[dtype] = dtypes.get(dtype, 0) + 1
        parameters += count
        total_bytes += count * {"float32": 4, "float64": 8, "int32": 4, "int64": 8}.get(dtype, 2)
    return {
        "name": os.path.basename(os.path.normpath(model_dir)),
        "architecture": arch.name,
        "tensor_count": len(source.names()),
        "parameter_count": parameters,
        "tensor_types": dtypes,
        "file_bytes": total_bytes,
        "context_limit": spec.max_position_embeddings,
        "layer_count": len(spec.layers),
        "scheduled_layers": len(spec.schedule),
        "vocab_size": spec.vocab_size,
        "hidden_size": spec.hidden_size,
        "tied_output": spec.head_name is None,
        "kv_bytes_per_token_bf16": planner.kv_bytes_per_token(spec, 2),
    }


def model_info(args: List[str]) -> int:
    found, places = _parse(args, "model-info", {}, {"--json"}, 1)
    if not places:
        raise UsageError("model-info needs a model path")
    report = _model_report(places[0])
    if found.get("json"):
        print(json.dumps(report, indent=2))
    else:
        for key, value in report.items():
            print(f"{key:24} {value}")
    return 0


def plan_memory(model_dir: str, ctx: int, batch: int, dtype: str, device_bytes: Optional[int],
                page_size: int = 16) -> dict:
    """The memory plan of the model in ``model_dir`` (its config.json is all that is read)."""
    from .config import load_config
    from .engine import planner

    arch, config = load_config(model_dir)
    return planner.plan_memory(arch.model_spec(config), ctx, batch, dtype, device_bytes, page_size)


def plan(args: List[str]) -> int:
    found, places = _parse(args, "plan", {"--ctx": ("ctx", int), "--batch": ("batch", int),
                                          "--dtype": ("dtype", str), "--kv-type": ("kv_type", str),
                                          "--device-bytes": ("device_bytes", int),
                                          "--page-size": ("page_size", int)}, {"--json"}, 1)
    if not places:
        raise UsageError("plan needs a model path")
    report = plan_memory(places[0], found.get("ctx", 2048), found.get("batch", 1),
                         found.get("dtype", "bfloat16"), found.get("device_bytes"), found.get("page_size", 16))
    if found.get("json"):
        print(json.dumps(report, indent=2))
    else:
        for key, value in report.items():
            print(f"{key:24} {value}")
    return 0 if report["feasible"] else InfeasibleError.exit_code


def random_weights(args: List[str]) -> int:
    found, places = _parse(args, "random-weights", {"--seed": ("seed", int), "--dtype": ("dtype", str)}, set(), 2)
    if len(places) != 2:
        raise UsageError("random-weights needs a config.json and an output folder")
    from .engine.loader import write_random_model

    with open(places[0], "r", encoding="utf-8") as handle:
        config = json.load(handle)
    write_random_model(places[1], config, found.get("seed", 0), found.get("dtype", "bfloat16"))
    print(f"wrote {places[1]}")
    return 0


def generate(args: List[str]) -> int:
    valued = {
        "--prompt": ("prompt", str), "--max-tokens": ("max_tokens", int), "--ctx": ("ctx", int),
        "--temperature": ("temperature", float), "--top-k": ("top_k", int), "--top-p": ("top_p", float),
        "--min-p": ("min_p", float), "--repetition-penalty": ("repetition_penalty", float),
        "--presence-penalty": ("presence_penalty", float), "--frequency-penalty": ("frequency_penalty", float),
        "--seed": ("seed", int), "--dtype": ("dtype", str), "--page-size": ("page_size", int),
        "--kv-type": ("kv_type", str), "--device": ("device", str),
    }
    found, places = _parse(args, "generate", valued, {"--json"}, 1)
    if not places:
        raise UsageError("generate needs a model path")
    if "prompt" not in found:
        raise UsageError("generate needs --prompt (token ids separated by spaces or commas)")
    try:
        prompt = [int(t) for t in found["prompt"].replace(",", " ").split()]
    except ValueError:
        raise InvalidArgumentError("--prompt takes token ids; this engine has no tokenizer") from None
    max_tokens = found.get("max_tokens", 32)
    if max_tokens < 1:
        raise InvalidArgumentError("--max-tokens must be at least 1")
    dtype = found.get("dtype", "bfloat16")
    kv_type = found.get("kv_type")
    if kv_type is not None and kv_type not in ("bf16", "bfloat16", "f32", "float32"):
        raise InvalidArgumentError(f"--kv-type {kv_type!r}: the cache has the run's dtype; quantized caches are not built")

    from .engine.engine import Engine
    from .sampling import SamplingParams

    params = SamplingParams(
        max_new_tokens=max_tokens, temperature=found.get("temperature", 0.0), top_k=found.get("top_k", 40),
        top_p=found.get("top_p", 0.95), min_p=found.get("min_p", 0.05),
        repetition_penalty=found.get("repetition_penalty", 1.0),
        presence_penalty=found.get("presence_penalty", 0.0),
        frequency_penalty=found.get("frequency_penalty", 0.0), seed=found.get("seed", 0))
    engine = Engine(places[0], dtype=dtype, device=found.get("device", "cuda:0"),
                    page_size=found.get("page_size", 16), ctx=found.get("ctx"), max_num_seqs=1)
    as_json = bool(found.get("json"))
    eos = set(engine.default_eos)

    def stream(request, token):
        if not as_json and token not in eos:
            print(token, end=" ", flush=True)

    started = time.time()
    result = engine.generate([prompt], params, on_token=stream)[0]
    elapsed = time.time() - started
    if as_json:
        print(json.dumps({
            "prompt_tokens": result.prompt_tokens, "reused_tokens": result.reused_tokens,
            "processed_tokens": result.processed_tokens, "generated_tokens": len(result.tokens),
            "finish": result.finish, "tokens": result.tokens,
            "tokens_per_second": len(result.tokens) / elapsed if elapsed > 0 else 0.0,
        }))
    else:
        print()
    return 0


COMMANDS = {"generate": generate, "model-info": model_info, "plan": plan, "random-weights": random_weights}


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        if not argv or argv[0] in ("-h", "--help", "help"):
            print(USAGE, end="")
            return 0 if argv else UsageError.exit_code
        command = COMMANDS.get(argv[0])
        if command is None:
            raise UsageError(f'unknown command "{argv[0]}"')
        return command(argv[1:])
    except ViperaError as error:
        print(f"vipera: {error.kind}: {error}", file=sys.stderr)
        if isinstance(error, UsageError):
            print(USAGE, end="", file=sys.stderr)
        return error.exit_code
    except Exception as error:  # a fault that is not one of the engine's own kinds is internal too
        if os.environ.get("VIPERA_TRACEBACK"):
            raise
        print(f"vipera: internal: {type(error).__name__}: {error}", file=sys.stderr)
        return InternalError.exit_code


if __name__ == "__main__":
    sys.exit(main())
