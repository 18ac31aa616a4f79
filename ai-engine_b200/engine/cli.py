"""The command line, in the manner of the reference's binary
(crates/ai-engine/src/cli.rs:10-26: `-c/--config <toml>`, `--check`), reduced to
what an engine without a server needs: token ids in, token ids out.

    ai-engine --model DIR [--config provider.toml|json] [--check]
              (--prompt-ids 1,2,3 | --prompt-file prompts.jsonl)
              [--max-tokens N] [--temperature T] [--top-k K] [--top-p P] [--seed S]
              [--ignore-eos] [--stats] [--profile [--peaks GB/s,TFLOP/s]]

The config file is the local-provider block of the reference's ai-engine.toml
(crates/ai-engine-config/src/lib.rs:97-140): either a `[[provider]]` table (the
first one whose kind is not a remote API) or a flat table, with the keys
weights_path, device, max_num_seqs, block_size, kv_cache_blocks, plus dtype,
kv_cache_gb, max_num_batched_tokens, max_seq_len, random_weights, seed,
norm_weight_std.  `${VAR}` is replaced from the environment and a missing
variable is an error (crates/ai-engine-config/src/interpolate.rs:5).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from typing import List


def interpolate_env(text: str) -> str:
    def sub(m):
        name = m.group(1)
        if name not in os.environ:
            raise ValueError(f"config: environment variable {name} is not set")
        return os.environ[name]

    return re.sub(r"\$\{([A-Za-z_][A-Za-z0-9_]*)\}", sub, text)


_IGNORED_PROVIDER_KEYS = {"id", "kind", "base_url", "api_key", "timeout_secs", "http2",
                          "extra_headers", "cluster", "engine", "pool_size"}


def read_provider_config(path: str) -> dict:
    with open(path) as f:
        text = interpolate_env(f.read())
    if path.endswith(".json"):
        raw = json.loads(text)
    else:
        import tomllib
        raw = tomllib.loads(text)
    if isinstance(raw.get("provider"), list):
        local = [p for p in raw["provider"] if p.get("kind") not in ("openai", "anthropic", "local-cluster")]
        if not local:
            raise ValueError(f"{path}: no local [[provider]] block")
        raw = local[0]
        if raw.get("engine") not in (None, "paged"):
            raise ValueError(f"{path}: engine `{raw['engine']}` is not built (only `paged`)")
    return {k: v for k, v in raw.items() if k not in _IGNORED_PROVIDER_KEYS}


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="ai-engine", description="Llama 3 on one B200: token ids in, token ids out")
    ap.add_argument("--model", help="model folder (config.json + *.safetensors); overrides weights_path")
    ap.add_argument("-c", "--config", help="provider-like options file (.toml or .json)")
    ap.add_argument("--check", action="store_true", help="validate the configuration and the model folder, then exit")
    ap.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids (repeatable)")
    ap.add_argument("--prompt-file", help="JSON lines, one list of token ids each")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--dtype", choices=["bf16", "fp32", "bfloat16", "float32"], default=None)
    ap.add_argument("--stats", action="store_true", help="print engine counters to stderr at the end")
    ap.add_argument("--profile", action="store_true",
                    help="time every kernel launch with CUDA events (eager launches, no graphs) and print "
                         "time, bytes, flops and roofline fraction per class of kernel to stderr")
    ap.add_argument("--peaks", default="7700,2250",
                    help="memory bandwidth in GB/s and bf16 TFLOP/s that --profile's fractions are taken "
                         "against (default: the B200's nominal 7700,2250)")
    return ap.parse_args(argv)


def check_only(options: dict) -> None:
    """Validate options, config.json and the tensors of the folder without a device."""
    from ..config.registry import load_config
    from ..parts.model import tensor_specs_of
    from ..weights.loader import ModelFolder, check_and_resolve
    from .engine import EngineOptions

    opts = EngineOptions.from_dict(options)
    opts.validate()
    if not opts.weights_path:
        raise ValueError("no model folder given (--model or weights_path)")
    arch, cfg = load_config(opts.weights_path)
    if not opts.random_weights:
        folder = ModelFolder(opts.weights_path)
        check_and_resolve(tensor_specs_of(arch.build_spec(cfg)),
                          {n: folder.info(n) for n in folder.names()}, where=opts.weights_path)
        folder.close()


def main(argv=None) -> int:
    args = parse_args(argv)
    try:
        options = read_provider_config(args.config) if args.config else {}
        if args.model:
            options["weights_path"] = args.model
        if args.dtype:
            options["dtype"] = args.dtype
        if args.check:
            check_only(options)
            print("ok")
            return 0
        prompts: List[List[int]] = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
        if args.prompt_file:
            with open(args.prompt_file) as f:
                prompts += [json.loads(l) for l in f if l.strip()]
        if not prompts:
            raise ValueError("no prompt: give --prompt-ids or --prompt-file")
        from ..sampling.params import SamplingParams
        from .engine import Engine

        if args.profile:
            from ..kernels import profile
            profile.start()
        engine = Engine(None, **options)
        sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            seed=args.seed, max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
        for out in engine.generate(prompts, sp):
            print(",".join(str(t) for t in out), flush=True)
        if args.profile:
            gbs, tf = (float(x) for x in args.peaks.split(","))
            print(profile.table(profile.stop(gbs, tf)), file=sys.stderr)
        if args.stats:
            print(json.dumps(engine.stats()), file=sys.stderr)
        return 0
    except Exception as e:  # one line for the user, like the reference's anyhow errors
        print(f"ai-engine: error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
