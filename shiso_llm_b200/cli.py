"""Command line: ``python -m shiso_llm_b200 generate|init-random|info``.

The reference ships only ``shiso serve`` (crates/shiso-server/src/cli.rs:31-47); its
engine options keep their names here where they exist there
(crates/shiso-runtime/src/options.rs:75-320): ``-m/--model``, ``-c/--ctx``,
``--max-num-seqs``, ``--kv-cache-tokens``, ``--max-num-batched-tokens``, and the sampling
knobs of its requests (crates/shiso-ir/src/request.rs:33-85): ``--temperature``,
``--top-k``, ``--top-p``, ``--min-p``, ``--seed``, ``--max-tokens``.  Prompts are token
ids: this engine has no tokenizer.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time


def preset_path(name: str) -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "config", "presets", name + ".json")


def preset_names() -> list[str]:
    d = os.path.dirname(preset_path("x"))
    return sorted(f[:-5] for f in os.listdir(d) if f.endswith(".json"))


def load_config_document(args) -> dict:
    if args.config:
        with open(args.config, "r", encoding="utf-8") as f:
            return json.load(f)
    path = preset_path(args.preset)
    if not os.path.isfile(path):
        raise SystemExit(f"unknown preset {args.preset!r}; available: {', '.join(preset_names())}")
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def init_random(document: dict, seed: int, out: str, storage_dtype: str = "bfloat16", std: float = 0.02,
                num_layers: int | None = None) -> None:
    """Writes a model folder (config.json, model.safetensors) from a configuration and a seed."""
    import torch

    from .config import plan_from_document
    from .parts import BuildEnv, Model
    from .weights import random_tensors, write_model_folder

    if num_layers is not None:
        document = dict(document)
        document["layer_types"] = list(document["layer_types"])[:num_layers]
        document["num_hidden_layers"] = num_layers
    _, _, plan = plan_from_document(document)
    model = Model(plan, BuildEnv(dtype=torch.float32, device=torch.device("cpu"), ops=None))
    write_model_folder(out, document, random_tensors(model.tensor_specs(), seed, std, storage_dtype))


def cmd_init_random(args) -> int:
    init_random(load_config_document(args), args.seed, args.out, args.storage_dtype, args.std, args.num_layers)
    print(f"wrote {args.out}")
    return 0


def cmd_info(args) -> int:
    from .config import load_config

    arch, config = load_config(args.model)
    plan = arch.build_plan(config)
    derived = {k: getattr(config, k) for k in ("intermediate_size", "head_dim") if hasattr(config, k)}
    print(json.dumps({"architecture": arch.name, "config": config.to_dict(), "derived": derived,
                      "layers": [layer.mixer.kind for layer in plan.layers]}, indent=2))
    return 0


def parse_prompts(args, vocab: int) -> list:
    prompts = []
    for text in args.prompt_ids or []:
        prompts.append([int(t) for t in text.replace(",", " ").split()])
    if args.prompt_len:
        import torch

        g = torch.Generator().manual_seed(args.prompt_seed)
        for n in args.prompt_len:
            prompts.append(torch.randint(0, vocab, (n,), generator=g).tolist())
    if not prompts:
        raise SystemExit("give --prompt-ids \"1,2,3\" (repeatable) or --prompt-len N (repeatable)")
    return prompts


class FrontierRows:
    """Writes the logits row at the end of every prompt - the row the request's first token is
    picked from - as ``DIR/<request>.f32.npy`` (float32 ``[vocab]``) plus ``DIR/index.json``, after
    the row dump of the reference's parity runner (crates/shiso-bench/src/bin/parity.rs:11-16).
    Like that one it refuses to replace anything already there."""

    def __init__(self, folder: str):
        self.folder = folder
        self.index = []
        os.makedirs(folder, exist_ok=True)
        if os.listdir(folder):
            raise SystemExit(f"--dump-logits {folder}: the folder is not empty; a dump replaces nothing")

    def __call__(self, plan, logits) -> None:
        import numpy as np

        row = 0
        for entry in plan.entries:
            if not entry.samples:
                continue
            request = entry.request
            if entry.start + entry.count == len(request.prompt) and not request.preemptions:
                name = f"{request.id}.f32.npy"
                np.save(os.path.join(self.folder, name), logits[row].detach().float().cpu().numpy())
                self.index.append({"request": request.id, "prompt_tokens": len(request.prompt),
                                   "position": len(request.prompt) - 1, "file": name})
            row += 1

    def close(self) -> None:
        with open(os.path.join(self.folder, "index.json"), "w", encoding="utf-8") as f:
            json.dump({"dtype": "float32", "rows": self.index}, f, indent=2)
            f.write("\n")


def cmd_generate(args) -> int:
    from .api import LLM
    from .sampling import SamplingParams

    if (args.model is None) == (args.random_config is None):
        raise SystemExit("give either -m/--model DIR or --random-config NAME")
    common = dict(
        dtype=args.dtype, ctx=args.ctx, page_size=args.page_size, kv_cache_tokens=args.kv_cache_tokens,
        gpu_memory_utilization=args.gpu_memory_utilization, max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_num_batched_tokens, cuda_graphs=not args.no_cuda_graphs, device=args.device,
        dump_layers=args.dump_layers,
    )
    if args.random_config is not None:
        # weights drawn on the device from the seed (the distribution of `init-random`, not its
        # numbers: that command draws on the host so that a folder is the same everywhere)
        import torch

        from .config import plan_from_document
        from .engine import Engine, EngineOptions
        from .engine.core import parse_dtype
        from .parts import BuildEnv, Model
        from .weights import random_device_tensors

        path = preset_path(args.random_config)
        if not os.path.isfile(path):
            raise SystemExit(f"unknown preset {args.random_config!r}; available: {', '.join(preset_names())}")
        with open(path, "r", encoding="utf-8") as f:
            _, _, plan = plan_from_document(json.load(f))
        specs = Model(plan, BuildEnv(dtype=torch.float32, device=torch.device("cpu"), ops=None)).tensor_specs()
        tensors = random_device_tensors(specs, args.weights_seed, parse_dtype(args.dtype), torch.device(args.device))
        engine = Engine.from_plan(plan, tensors, EngineOptions(**common))
        llm = LLM(engine, prefill_chunk=args.prefill_chunk, on_exhaustion=args.on_exhaustion, lookahead=not args.no_lookahead)
    else:
        llm = LLM(args.model, prefill_chunk=args.prefill_chunk, on_exhaustion=args.on_exhaustion,
                  lookahead=not args.no_lookahead, **common)
    prompts = parse_prompts(args, llm.engine.vocab_size)
    params = SamplingParams(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p, seed=args.seed,
        max_new_tokens=args.max_tokens, stop_token_ids=tuple(args.stop_token_ids or ()), ignore_eos=args.ignore_eos,
        bad_token_ids=tuple(args.bad_token_ids or ()),
    )
    rows = FrontierRows(args.dump_logits) if args.dump_logits else None
    llm.logits_tap = rows
    profiler = llm.engine.enable_launch_profile(args.profile_dir) if args.profile_dir else None
    started = time.time()
    outputs = llm.generate(prompts, params)
    elapsed = time.time() - started
    if rows is not None:
        rows.close()
    if profiler is not None:
        llm.engine.disable_launch_profile()
        profiler.write()
        print(profiler.text(), file=sys.stderr)
    for out in outputs:
        print(json.dumps({"request": out.request_id, "prompt_tokens": len(out.prompt_token_ids),
                          "token_ids": out.token_ids, "finish_reason": out.finish_reason, "error": out.error}))
    produced = sum(len(o.token_ids) for o in outputs)
    print(f"# {produced} tokens in {elapsed:.3f} s ({produced / max(elapsed, 1e-9):.1f} tok/s), "
          f"stats {llm.scheduler.stats}", file=sys.stderr)
    return 0


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="shiso_llm_b200", description=__doc__.split("\n\n")[0])
    sub = parser.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids for token-id prompts")
    g.add_argument("-m", "--model", help="model folder (config.json + *.safetensors)")
    g.add_argument("--random-config", metavar="NAME", help=f"instead of a folder: random weights of a preset ({', '.join(preset_names())})")
    g.add_argument("--weights-seed", type=int, default=0, help="seed of --random-config's weights")
    g.add_argument("--prompt-ids", action="append", help="comma- or space-separated token ids; repeatable")
    g.add_argument("--prompt-len", action="append", type=int, help="a uniform-random prompt of this length; repeatable")
    g.add_argument("--prompt-seed", type=int, default=0)
    g.add_argument("--max-tokens", type=int, default=16, help="new tokens per request")
    g.add_argument("--temperature", type=float, default=0.0, help="<= 0 is greedy")
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--stop-token-ids", type=int, nargs="*")
    g.add_argument("--bad-token-ids", type=int, nargs="*", help="token ids that are never emitted")
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    g.add_argument("-c", "--ctx", type=int, default=4096)
    g.add_argument("--page-size", type=int, default=16)
    g.add_argument("--kv-cache-tokens", type=int, default=None, help="tokens the cache pool holds (default: max-num-seqs x ctx)")
    g.add_argument("--gpu-memory-utilization", type=float, default=None,
                   help="instead: the share of device memory this process may fill; the pool gets what is left of it")
    g.add_argument("--max-num-seqs", type=int, default=4)
    g.add_argument("--max-num-batched-tokens", type=int, default=2048)
    g.add_argument("--prefill-chunk", type=int, default=None)
    g.add_argument("--on-exhaustion", choices=["preempt", "fail"], default="preempt")
    g.add_argument("--no-cuda-graphs", action="store_true", help="launch decode steps kernel by kernel")
    g.add_argument("--no-lookahead", action="store_true",
                   help="wait for each step's tokens on the host before planning the next step")
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--dump-logits", metavar="DIR", help="write the logits row at the end of every prompt to DIR")
    g.add_argument("--dump-layers", type=int, choices=[0, 1, 2], default=0,
                   help="print statistics of the residual stream after every layer (2: after every mixer and feed-forward) to stderr")
    g.add_argument("--profile-dir", metavar="DIR",
                   help="time every kernel launch of every step (steps then run kernel by kernel) and write launches.json / launches.txt to DIR")
    g.set_defaults(func=cmd_generate)

    r = sub.add_parser("init-random", help="write a model folder with random weights")
    r.add_argument("--preset", default="lfm2-1.2b", help=f"one of: {', '.join(preset_names())}")
    r.add_argument("--config", help="a config.json to use instead of a preset")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--storage-dtype", choices=["bfloat16", "float32", "float16"], default="bfloat16")
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--num-layers", type=int, default=None, help="keep only the first N layers")
    r.set_defaults(func=cmd_init_random)

    i = sub.add_parser("info", help="print a model folder's configuration and layer kinds")
    i.add_argument("-m", "--model", required=True)
    i.set_defaults(func=cmd_info)
    return parser


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return args.func(args)
