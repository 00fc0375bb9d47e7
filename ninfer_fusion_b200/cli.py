"""Command line front ends: `python -m ninfer_fusion_b200.cli {generate,serve,inspect,make-artifact,perplexity}`.

One loader builds the engine for every front end: weights come from a `.ninfer` artifact (tensors are
materialised onto the device, quantised formats are decoded or re-encoded for the tcgen05 quantised GEMMs) or
are random-initialised for a registered geometry; the tokenizer comes from the artifact's embedded
`tokenizer.json`, from a file, or is a small byte-level BPE when neither exists.

Reference: apps/cli/main.cpp + options.cpp (usage block README.md:391-429), apps/serve/main.cpp,
apps/perplexity (corpus scoring), src/serve/serve_options.cpp (docs/serving.md:658-705).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time
from typing import Dict, Optional, Tuple

import torch

from .artifact import layouts as L
from .artifact.container import ArtifactReader, ArtifactWriter
from .frontend.chat import BUILTIN_TEMPLATE, renderer_for
from .frontend.tokenizer import Tokenizer
from .models.config import ModelConfig, get_config
from .models.weights import QUANT_LEAVES, quantize_weights, random_weights, total_bytes
from .ops.groupint import GroupIntWeight
from .runtime.engine import Engine, RequestOptions
from .runtime.program import ReferenceProgram, SamplingParams

DEFAULT_CORPUS = ("The quick brown fox jumps over the lazy dog. Hello world! def main(): return 0\n"
                  "<|im_start|>user\nWhat is 2 + 2?<|im_end|>\n<|im_start|>assistant\n4<|im_end|>\n") * 8
SPECIAL_TOKENS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>",
                  "<tool_response>", "</tool_response>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>"]


def add_model_args(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--artifact", help=".ninfer artifact (weights + embedded tokenizer / chat template)")
    ap.add_argument("--model", default="tiny-dense", help="registered geometry for --random-init (see models/config.py); an "
                    "attention-only package (spark-x2.5-4b, muse-glimmer-30b, gemma4-31b, optionally NAME@LAYERS) runs on "
                    "the CPU oracle at a reduced debug geometry unless --full-geometry is given")
    ap.add_argument("--full-geometry", action="store_true", help="attention-only packages: the full widths and vocabulary")
    ap.add_argument("--random-init", action="store_true", help="random weights of --model instead of an artifact")
    ap.add_argument("--layers", type=int, default=0, help="shrink the geometry to this many layers (debug)")
    ap.add_argument("--tokenizer", help="tokenizer.json (overrides the artifact's embedded one)")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "fp8", "nvfp4", "q4", "q5", "q6", "w8", "q4+h64", "q4+h128", "q5+h64", "q6+h64", "w8+h64", "stored"],
                    help="matmul weight format on the device; q4/q5/q6/w8 keep groupwise-int codes and dequantise in the "
                         "decode kernels ('+h64': input dimension rotated by a block Hadamard first); 'stored' keeps an artifact's groupwise-int tensors exactly as encoded")
    ap.add_argument("--kv-descent-age", type=int, default=0,
                    help="with --kv-dtype mixed: cells whose newest token is older than this many tokens descend one "
                         "precision rung per pass (bf16 -> fp8 -> nvfp4); 0 = no automatic descent")
    ap.add_argument("--kv-descent-target-mib", type=float, default=0.0,
                    help="stop descending once the live KV cells of the mixed layers fit in this many MiB (0 = no target)")
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "fp8", "fp8h", "int8", "nvfp4", "mixed"],
                    help="KV cache codec (fp8h = fp8 per-row with K in the Hadamard frame)")
    ap.add_argument("--kv-descent-floor-nats", type=float, default=0.0,
                    help="with --kv-descent-target-mib: solve the whole per-cell allocation every pass (cells may be "
                         "assigned several rungs down at once) and never spend more than this total precision loss; a "
                         "target that cannot be reached inside it moves nothing (0: the incremental one-rung walk)")
    ap.add_argument("--kv-descent-rung-nats", default="0.01,0.08",
                    help="measured loss, in nats per cell, of a cell entering fp8 and nvfp4")
    ap.add_argument("--kv-tier-formats", default="",
                    help="with --kv-dtype mixed: hot=<tier>,tail=<tier>,cold=<tier> over bf16 / fp8 / nvfp4: new pages "
                         "start in the hot tier, cells descend no further than the cold tier")
    ap.add_argument("--kv-layer-spec", default="", help="per-layer KV storage, e.g. 'all:fp8' or '0-3:bf16,4-15:nvfp4'")
    ap.add_argument("--kv-bits", type=float, default=None,
                    help="one ceiling on the average bits per KV element: the bit-budget planner picks a tier per layer")
    ap.add_argument("--kv-k-bits", type=float, default=None, help="ceiling of the K planes (with --kv-v-bits)")
    ap.add_argument("--kv-v-bits", type=float, default=None, help="ceiling of the V planes (with --kv-k-bits)")
    ap.add_argument("--kv-bits-mode", default=None, choices=["joint", "split", "ceiling"],
                    help="split: each plane is layered on its own ceiling and a layer both planes cannot share is refused "
                         "by index; ceiling: deploy min(k, v) on both planes and report the unspendable headroom")
    ap.add_argument("--kv-tier-scores", default="", help="tier=penalty table replacing the ladder's priors (see "
                                                         "`python -m ninfer_fusion_b200.kv.kv_bits score-table show`)")
    ap.add_argument("--kv-k-tier-scores", default="", help="score table of the K planes (split reading)")
    ap.add_argument("--kv-v-tier-scores", default="", help="score table of the V planes (split reading)")
    ap.add_argument("--max-context", type=int, default=4096)
    ap.add_argument("--max-lanes", type=int, default=8, help="concurrent sequences")
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--prefill-chunk-mode", default=None, choices=["dynamic", "manual"],
                    help="dynamic: the bandwidth governor shrinks / restores the prefill unit and its share against "
                         "decode latency (default; NINFER_FT_BW_GOV=0 in the environment selects manual); manual: the "
                         "unit stays --prefill-chunk.  NINFER_FT_BW_TRACE=1 prints every change")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--no-graphs", action="store_true", help="eager decode instead of CUDA graphs")
    ap.add_argument("--spec", default="none", choices=["none", "off", "auto", "mtp", "dflash", "dspark"],
                    help="speculative decoding: mtp = the draft module proposes; auto = mtp when the weights carry a "
                         "draft module; none / off = ordinary decode")
    ap.add_argument("--draft-tokens", type=int, default=0,
                    help="drafts per round, 1..15; 0 with --spec mtp = adaptive (the width follows acceptance and round "
                         "cost over a ladder of captured widths)")
    ap.add_argument("--spec-stochastic", action="store_true",
                    help="with --spec mtp and sampled requests: the draft module samples its proposals and the verifier "
                         "accepts with min(1, p / q) (general speculative sampling) instead of arg-max proposals")
    ap.add_argument("--spec-adaptive-width", action="store_true",
                    help="with --spec mtp: the number of drafts per round follows measured acceptance and round cost "
                         "(a ladder of widths up to --draft-tokens, one captured round per width)")
    ap.add_argument("--draft-head", default="",
                    help="with --spec mtp: shortlist draft head, either a count N (token ids 0..N-1) or a file of token "
                         "ids (one per line, or a .npy / .pt tensor); the target still verifies with the full head")
    ap.add_argument("--allow-unknown-template", action="store_true")
    ap.add_argument("--weight-budget-gib", type=float, default=0.0,
                    help="device bytes for weights; layers beyond it rotate in from pinned host memory (eager decode)")
    ap.add_argument("--vision", action="store_true",
                    help="attach the vision tower (the artifact's vision/ tensors, or random ones with --random-init)")
    ap.add_argument("--vision-layers", type=int, default=0, help="shrink the vision tower to this many blocks (debug)")
    ap.add_argument("--kv-capacity", default="full", help="main KV pool: 'full', 'auto' or a token count >= --max-context")
    ap.add_argument("--kv-headroom-gib", type=float, default=2.0, help="device memory left free by --kv-capacity auto")
    ap.add_argument("--planner", default="lru",
                    help="which cached frontier is given up under memory pressure: 'lru' (least recently used), or the "
                         "materialisation planner with a machine cost preset: b200 | h100 | rtx5090 | file:<path> "
                         "(a file measured on this machine by `python -m ninfer_fusion_b200.utils.calib`)")
    ap.add_argument("--cold-policy", default="none", choices=["none", "off", "host", "disk", "host-then-disk", "host+disk"],
                    help="where session frontiers go when the device pool needs their pages: pinned host memory, files, "
                         "or host first with files as its overflow (none: they are dropped)")
    ap.add_argument("--cold-host-bytes", default="0", help="pinned host budget, N[k|m|g]")
    ap.add_argument("--cold-disk-path", default="", help="directory of the file tier")
    ap.add_argument("--cold-disk-bytes", default="0", help="file tier budget, N[k|m|g]")
    ap.add_argument("--cold-entropy", action="store_true", help="entropy-code frontiers written to the file tier")
    ap.add_argument("--cold-journal", action="store_true",
                    help="keep the file tier's frontier -> file map in a journal inside --cold-disk-path and adopt the frontiers "
                         "a previous process left there (bound to the program, the model, the KV storage and the weights)")
    ap.add_argument("--cold-journal-flush", default="none", choices=["none", "flush", "fsync"],
                    help="what is forced after every journal record (the journal is a mirror: losing its tail costs a re-prefill)")
    ap.add_argument("--cold-read-gbs", type=float, default=0.0,
                    help="measured read rate of the file tier in GB/s; with --cold-prefill-tok-s a frontier is read back "
                         "only when that beats prefilling its tokens again (0 = always read back)")
    ap.add_argument("--cold-prefill-tok-s", type=float, default=0.0, help="measured prefill rate in tokens/s for that comparison")
    ap.add_argument("--cold-slots", action="store_true",
                    help="int8 KV pages leave the device as requantised cold slots (lossy, 0.55 of the bytes)")
    ap.add_argument("--anchor-interval", type=int, default=0,
                    help="keep a recovery frontier every N prompt tokens of a session's long prefill (0 = off)")
    ap.add_argument("--kv-rowscale", default=None,
                    help="K row-scale table (default: NINFER_KV_ROWSCALE, else <artifact>.kvrowscale.bin when present)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tp", type=int, default=1,
                    help="tensor-parallel ranks; launch the command with `python -m torch.distributed.run --nproc-per-node N "
                         "--master-addr 127.0.0.1 -m ninfer_fusion_b200.cli ...`: rank 0 serves, the others follow its steps")
    ap.add_argument("--ep", type=int, default=1,
                    help="expert-parallel ranks (MoE models): routed experts are split over the ranks, every request's "
                         "attention / GDN work lives on one rank, the ranks run in lock step; launch like --tp")
    ap.add_argument("--dp", type=int, default=1,
                    help="data-parallel ranks: independent replicas of the model behind one front end; launch like --tp")
    ap.add_argument("--rank-timeout", type=float, default=60.0,
                    help="seconds after which a silent rank fails the engine (control channel time-out)")


def _oracle_package(args):
    """The attention-only package --model names (random-init runs only: their checkpoints have no converter here)."""
    from .models.packages import GDN, PACKAGES, construct_oracle
    base = str(getattr(args, "model", "")).split("@")[0]
    if base not in PACKAGES or PACKAGES[base].count(GDN) or PACKAGES[base].config is not None:
        return None
    # random-init debug geometry: a few layers, a small vocabulary, narrow widths unless the caller asks for all of it
    full = bool(getattr(args, "full_geometry", False))
    return construct_oracle(args.model, layers=int(getattr(args, "layers", 0) or 0) or (0 if full else 4),
                            vocab=0 if full else 2048, hidden_div=1 if full else 8)


def load_model(args) -> Tuple[ModelConfig, Dict[str, object], Tokenizer, str]:
    tok: Optional[Tokenizer] = None
    template: Optional[str] = None
    if args.artifact and not args.random_init:
        with ArtifactReader(args.artifact) as rd:
            model_id, weights_id = rd.identity
            cfg = get_config(model_id)
            weights = {}
            from .utils.progress import Progress
            names = list(rd.tensors())
            bar = Progress(sum(rd.by_name[n].bytes for n in names), "loading")
            for name in names:
                o = rd.by_name[name]
                bar.advance(o.bytes, name)
                if (args.weights == "stored" and args.device != "cpu" and o.format in L.GROUP_FORMATS and len(o.shape) == 2
                        and name.rsplit("/", 1)[-1] in QUANT_LEAVES and "/moe/" not in name):
                    # zero-copy in format: the encoded object goes to the device as it is
                    raw = torch.frombuffer(bytearray(rd.payload(name)), dtype=torch.uint8)
                    weights[name] = GroupIntWeight(o.format, raw.to(args.device), o.shape)
                else:
                    weights[name] = rd.tensor(name)
            bar.close()
            if "tokenizer.json" in rd.by_name:
                tok = Tokenizer.from_json(rd.resource("tokenizer.json"))
            if "chat_template.jinja" in rd.by_name:
                template = rd.resource("chat_template.jinja").decode("utf-8")
        weights = {k: (v.to(torch.bfloat16) if torch.is_tensor(v) and v.dtype == torch.float32
                       and not k.endswith(("A_log", "dt_bias")) else v) for k, v in weights.items()}
        weights = {k: (v.to(args.device) if torch.is_tensor(v) else v) for k, v in weights.items()}
        name = f"{model_id}:{weights_id}"
    elif _oracle_package(args) is not None:
        # an attention-only package: served on the CPU by its fp32 oracle (the GPU gate names what the kernels lack)
        from .models.all_attention import package_model_config, random_package_weights
        pkg = _oracle_package(args)
        if str(args.device) != "cpu":
            from .models.packages import PACKAGES
            raise SystemExit(f"{pkg.model_id}: the GPU runtime lacks {', '.join(PACKAGES[pkg.model_id.split('@')[0]].missing())}; "
                             f"--device cpu runs the package on its oracle")
        args._package = pkg
        cfg = package_model_config(pkg, args.max_context)
        weights = random_package_weights(pkg, seed=args.seed)
        name = f"{pkg.model_id}:random-init"
    else:
        cfg = get_config(args.model)
        if args.layers:
            cfg = cfg.shrink(args.layers)
        weights = random_weights(cfg, args.device, seed=args.seed, std=0.05 if cfg.hidden <= 512 else 0.02,
                                 with_mtp=getattr(args, "spec", "none") == "mtp")
        name = f"{cfg.name}:random-init"
    renderer_for(template, allow_unknown=args.allow_unknown_template)  # refuses an unknown template early
    if args.weights not in ("bf16", "stored") and int(getattr(args, "tp", 1)) <= 1:   # (--tp: each rank quantises its shard)
        if args.device == "cpu":
            raise SystemExit("--weights fp8/nvfp4 needs a GPU (the CPU program runs the fp32 oracle)")
        weights = quantize_weights(weights, args.weights)
    if args.tokenizer:
        tok = Tokenizer.from_file(args.tokenizer)
    if tok is None:
        tok = Tokenizer.train_toy(DEFAULT_CORPUS, n_merges=min(200, max(0, cfg.vocab - 256 - len(SPECIAL_TOKENS))),
                                  added_tokens=SPECIAL_TOKENS)
    if tok.vocab_size > cfg.vocab:
        raise SystemExit(f"tokenizer has {tok.vocab_size} ids but the model's vocabulary is {cfg.vocab}")
    if getattr(args, "vision", False) and not any(k.startswith("vision/") for k in weights):
        if not args.random_init:
            raise SystemExit("--vision: the artifact has no vision/ tensors")
        from .models.vision import random_vision_weights
        weights.update(random_vision_weights(vision_config(args, cfg), args.device, seed=args.seed + 1))
    return cfg, weights, tok, name


def vision_config(args, cfg: ModelConfig):
    from .models.vision import VisionConfig
    base = VisionConfig()
    return base.scaled(args.vision_layers or base.layers, cfg.hidden)


def attach_vision(args, cfg: ModelConfig, weights, program):
    """Gives `program` the vision tower when --vision is set (device tower on a GPU program, fp32 oracle on the CPU)."""
    if not getattr(args, "vision", False):
        return program
    vcfg = vision_config(args, cfg)
    vw = {k: v for k, v in weights.items() if k.startswith("vision/")}
    if isinstance(program, ReferenceProgram):
        program.attach_vision(vcfg, vw)
    elif hasattr(program, "attach_vision"):
        from .models.vision import VisionTower
        program.attach_vision(VisionTower(vcfg, vw, args.device))
    else:
        raise SystemExit("--vision is not available with this program (speculative decoding)")
    return program


def setup_ranks(args):
    """Joins the rank group of a multi-GPU run: picks this rank's GPU, starts NCCL (bootstrap of the symmetric
    buffers) and the gloo control channel of the replicated engine.  Returns None for a single rank, else
    (rank, world, channel).  Must run before the model is loaded: it decides `args.device`."""
    from .parallel.replicated import RankChannel, world_from_env
    rank, world = world_from_env()
    plans = {k: max(int(getattr(args, k, 1)), 1) for k in ("tp", "ep", "dp")}
    if sum(1 for v in plans.values() if v > 1) > 1:
        raise SystemExit("give one of --tp, --ep and --dp")
    want = max(plans.values())
    if world == 1 and want == 1:
        return None
    if world != want:
        flag = max(plans, key=plans.get)
        raise SystemExit(f"--{flag} {want} needs {want} ranks (python -m torch.distributed.run --nproc-per-node {want} "
                         f"--master-addr 127.0.0.1 -m ninfer_fusion_b200.cli ...); found {world}")
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    args.device = f"cuda:{local}"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device(args.device))
    return rank, world, RankChannel.create(rank, world, timeout_s=float(getattr(args, "rank_timeout", 60.0)))


def check_device_routes(args, weights) -> None:
    """Refuses, before any kernel runs, a GPU without the instruction families of this package's kernels or a weight
    format without a route on it (archcaps.py); a CPU device runs the reference model and needs no route."""
    if not str(args.device).startswith("cuda"):
        return
    from . import archcaps
    major, minor = torch.cuda.get_device_capability(torch.device(args.device))
    formats, experts = set(), set()
    for name, t in weights.items():
        qt = getattr(t, "qtype", None)
        if qt == 1:
            fmt = "FP8_E4M3FN_ROW_BF16S"
        elif qt == 2:
            fmt = "NVFP4"
        elif qt is not None:
            fmt = getattr(t, "fmt", None)          # groupwise-int objects carry their artifact format name
        else:
            fmt = "BF16" if getattr(t, "dtype", None) == torch.bfloat16 else None
        if fmt is None or getattr(t, "dim", lambda: 2)() < 2 and qt is None:
            continue
        (experts if "/experts_" in name else formats).add(fmt)
    try:
        archcaps.require_artifact_formats_supported(formats, major * 10 + minor, experts)
    except archcaps.RouteRefused as e:
        raise SystemExit(f"this GPU cannot run the model: {e}")


def build_engine(args, cfg: ModelConfig, weights, ranks=None) -> Optional[Engine]:
    """The engine of this process.  With `ranks` (see setup_ranks) the model is tensor-parallel: rank 0 gets an
    Engine whose Program mirrors every step to the followers; a follower runs its loop here until the leader
    stops it and gets None."""
    kv = args.kv_dtype
    check_device_routes(args, weights)
    _kv_spec_from_ceilings(args, cfg)
    if ranks is not None and max(int(getattr(args, "ep", 1)), int(getattr(args, "dp", 1))) > 1:
        # every request lives on one rank (parallel/partitioned.py); expert parallelism adds the MoE exchange between
        # the ranks inside every forward pass, hence lock step
        from .parallel.partitioned import PartitionedLeader, partitioned_follower_loop
        rank, world, channel = ranks
        ep = int(getattr(args, "ep", 1)) > 1
        if getattr(args, "spec", "none") not in ("none", "off") or getattr(args, "vision", False) or args.weight_budget_gib > 0:
            raise SystemExit("--ep / --dp do not combine with --spec, --vision or --weight-budget-gib yet")
        if ep and cfg.moe is None:
            raise SystemExit("--ep shards routed experts: the model has none (use --dp for replicas of a dense model)")
        if args.kv_layer_spec:
            from .kv.policy import parse_layer_storage
            kv = parse_layer_storage(args.kv_layer_spec, len(cfg.attn_layers))
        if ep:
            # a rank that captures a decode graph runs warm-up passes the other ranks do not run: graphs would break
            # the lock step unless every rank captured the same ladder at the same moment, so EP serving runs eager
            args.no_graphs = True
        inner_factory = program_factory(args, cfg, weights, kv)

        def make_inner():
            prog = inner_factory()
            if ep:
                prog.model.ep = (rank, world, None)     # this rank's contiguous range of experts; the rest is replicated
            return prog
        if rank != 0:
            partitioned_follower_loop(make_inner(), channel, lockstep=ep)
            return None
        return Engine(lambda: PartitionedLeader(make_inner(), channel, args.max_lanes, lockstep=ep),
                      prefill_chunk=args.prefill_chunk, prefill_chunk_mode=getattr(args, "prefill_chunk_mode", None))
    if ranks is not None:
        from .parallel.replicated import LeaderProgram, follower_loop
        from .parallel.tp import TensorParallel
        rank, world, channel = ranks
        if getattr(args, "spec", "none") not in ("none", "off") or getattr(args, "vision", False) or args.weight_budget_gib > 0:
            raise SystemExit("--tp does not combine with --spec, --vision or --weight-budget-gib yet")
        if args.kv_layer_spec:
            from .kv.policy import parse_layer_storage
            kv = parse_layer_storage(args.kv_layer_spec, len(cfg.attn_layers))
        comm = TensorParallel(cfg, rank, world, args.device, max_tokens=max(args.prefill_chunk, args.max_lanes),
                              mode=TensorParallel.best_mode(world))
        text = {k: v for k, v in weights.items() if not k.startswith("vision/")}
        if any(hasattr(v, "qtype") for v in text.values()):
            raise SystemExit("--tp: give bf16 weights (every rank quantises its own shard: --weights applies after the split)")
        shard_w = comm.shard(text)
        if args.weights == "bf16" and comm.mode == "fused":
            shard_w = comm.fold_norms(dict(shard_w))
        elif args.weights not in ("stored", "bf16"):
            shard_w = quantize_weights(shard_w, args.weights)
        inner_factory = program_factory(args, cfg, shard_w, kv, shard=comm.geometry, comm=comm)
        if rank != 0:
            follower_loop(inner_factory(), channel)
            return None
        return Engine(lambda: LeaderProgram(inner_factory(), channel), prefill_chunk=args.prefill_chunk,
                      prefill_chunk_mode=getattr(args, "prefill_chunk_mode", None))
    if args.kv_layer_spec:
        from .kv.policy import parse_layer_storage
        kv = parse_layer_storage(args.kv_layer_spec, len(cfg.attn_layers))
    from .runtime.spec_options import from_strings
    try:
        head_ids = _draft_head_ids(getattr(args, "draft_head", ""), cfg)
        if head_ids is None and "text/draft_head_token_ids" in weights:
            head_ids = [int(v) for v in weights["text/draft_head_token_ids"].reshape(-1)]
        spec = from_strings(getattr(args, "spec", "none"), getattr(args, "draft_tokens", 0),
                            "shortlist" if getattr(args, "draft_head", "") else "auto", None,
                            getattr(args, "spec_stochastic", False))
        spec = spec.resolve("mtp/fc" in weights, "dflash/feature_proj" in weights, head_ids is not None)
    except ValueError as e:
        raise SystemExit(str(e)) from None
    if spec.backend == "dflash":
        raise SystemExit("--spec dflash: the engine's lanes draft with the MTP module; the DFlash drafter runs in the "
                         "static-batch generator (bench.py --spec dflash)")
    if spec.backend == "mtp":
        if not str(args.device).startswith("cuda"):
            raise SystemExit("--spec mtp needs a GPU")
        from .runtime.speculative import SpeculativeProgram
        adaptive = (spec.adaptive or getattr(args, "spec_adaptive_width", False)) and not spec.stochastic_drafts
        width = spec.width if adaptive or spec.draft_tokens else 3   # sampled drafts keep one width: three unless told

        def factory():
            return SpeculativeProgram(cfg, weights, args.device, max_lanes=args.max_lanes, max_context=args.max_context,
                                      draft_tokens=width, kv_format=kv, page_size=args.page_size,
                                      prefill_chunk=args.prefill_chunk, use_graph=not getattr(args, "no_graphs", False),
                                      stochastic_drafts=spec.stochastic_drafts,
                                      adaptive_width=adaptive,
                                      draft_head_ids=head_ids if spec.proposal_head == "shortlist" else None)
        return Engine(factory, prefill_chunk=args.prefill_chunk,
                      prefill_chunk_mode=getattr(args, "prefill_chunk_mode", None))
    return Engine(program_factory(args, cfg, weights, kv), prefill_chunk=args.prefill_chunk,
                      prefill_chunk_mode=getattr(args, "prefill_chunk_mode", None))


def parse_bytes(text: str) -> int:
    """'N', 'Nk', 'Nm', 'Ng' (binary multiples) -> bytes.  Anything else is refused, not read as zero."""
    t = str(text).strip().lower()
    mult = {"k": 1 << 10, "m": 1 << 20, "g": 1 << 30}.get(t[-1:], 1)
    num = t[:-1] if t[-1:] in "kmg" else t
    try:
        v = float(num)
    except ValueError:
        raise SystemExit(f"'{text}' is not a byte count (N, Nk, Nm or Ng)") from None
    if v < 0:
        raise SystemExit(f"'{text}' is negative")
    return int(v * mult)


def apply_cold_policy(args, prog) -> None:
    """--cold-policy / --cold-host-bytes / --cold-disk-path / --cold-disk-bytes: where frontiers that are pushed out
    of the device pool go (pinned host memory first, files as its overflow, dropped otherwise)."""
    policy = getattr(args, "cold_policy", "none") or "none"
    policy = {"off": "none", "host+disk": "host-then-disk"}.get(policy, policy)
    host_b = parse_bytes(getattr(args, "cold_host_bytes", "0") or "0")
    disk_b = parse_bytes(getattr(args, "cold_disk_bytes", "0") or "0")
    path = getattr(args, "cold_disk_path", "") or ""
    if policy == "none":
        if host_b or disk_b or path:
            raise SystemExit("--cold-host-bytes / --cold-disk-* need --cold-policy host | disk | host-then-disk")
        if getattr(args, "cold_journal", False) or getattr(args, "cold_read_gbs", 0.0) or getattr(args, "cold_prefill_tok_s", 0.0):
            raise SystemExit("--cold-journal / --cold-read-gbs / --cold-prefill-tok-s need a file tier (--cold-policy disk | host-then-disk)")
        return
    if policy in ("host", "host-then-disk") and host_b <= 0:
        raise SystemExit(f"--cold-policy {policy} needs --cold-host-bytes")
    if policy in ("disk", "host-then-disk") and (not path or disk_b <= 0):
        raise SystemExit(f"--cold-policy {policy} needs --cold-disk-path and --cold-disk-bytes")
    if not hasattr(prog, "host_budget_bytes"):
        raise SystemExit("this program keeps no frontiers: --cold-policy does not apply")
    # the disk tier is fed from the host tier: with the plain `disk` policy the host tier is only a staging page
    prog.host_budget_bytes = host_b if policy != "disk" else max(host_b, 1)
    if policy in ("disk", "host-then-disk"):
        prog.cold_dir, prog.disk_budget_bytes = path, disk_b
        prog.cold_entropy = bool(getattr(args, "cold_entropy", False))
    journal = bool(getattr(args, "cold_journal", False))
    read_gbs, tok_s = float(getattr(args, "cold_read_gbs", 0.0) or 0.0), float(getattr(args, "cold_prefill_tok_s", 0.0) or 0.0)
    if (journal or read_gbs or tok_s) and policy not in ("disk", "host-then-disk"):
        raise SystemExit("--cold-journal / --cold-read-gbs / --cold-prefill-tok-s need a file tier (--cold-policy disk | host-then-disk)")
    if (read_gbs > 0) != (tok_s > 0):
        raise SystemExit("--cold-read-gbs and --cold-prefill-tok-s are given together")
    if read_gbs > 0:
        from .runtime.cold_journal import RecallCost
        prog.recall_cost = RecallCost(read_gbs=read_gbs, prefill_tok_s=tok_s)
    if journal:
        rep = prog.enable_cold_journal(weights_id=_weights_identity(args), flush=getattr(args, "cold_journal_flush", "none"))
        print(f"[cold-journal] adopted {rep['adopted']} frontiers ({rep['records']} records, {len(rep['holes'])} holes, "
              f"{rep['orphans_removed']} orphan files removed)" + (f"; previous journal refused: {rep['refused']}" if rep["refused"] else ""),
              file=sys.stderr, flush=True)


def _weights_identity(args) -> str:
    """What names the set of weights a cold copy was computed with: the artifact file (path, size, modification time) or
    the seed of random weights."""
    art = getattr(args, "artifact", None)
    if art:
        try:
            st = os.stat(art)
            return f"artifact:{os.path.abspath(art)}:{st.st_size}:{int(st.st_mtime)}"
        except OSError:
            return f"artifact:{art}"
    return f"random:{getattr(args, 'model', '')}:{getattr(args, 'seed', 0)}:{getattr(args, 'weights', '')}"


def _kv_spec_from_ceilings(args, cfg: ModelConfig) -> None:
    """--kv-bits / --kv-k-bits + --kv-v-bits -> the per-layer storage spec (kv/kv_bits.py); fills args.kv_layer_spec."""
    bits, kb, vb = getattr(args, "kv_bits", None), getattr(args, "kv_k_bits", None), getattr(args, "kv_v_bits", None)
    tables = [getattr(args, n, "") for n in ("kv_tier_scores", "kv_k_tier_scores", "kv_v_tier_scores")]
    if bits is None and kb is None and vb is None:
        if any(tables) or getattr(args, "kv_bits_mode", None):
            raise SystemExit("--kv-tier-scores / --kv-bits-mode steer the bit-budget planner: give --kv-bits or the two "
                             "per-plane ceilings")
        return
    if args.kv_layer_spec:
        raise SystemExit("--kv-layer-spec names the tiers itself; a bit ceiling would compute them: give one of the two")
    from .kv import kv_bits as KB

    def load(path):
        if not path:
            return None
        with open(path) as f:
            return KB.parse_scores(f.read(), path)
    try:
        plan = KB.resolve(len(cfg.attn_layers), bits, kb, vb, getattr(args, "kv_bits_mode", None), *(load(t) for t in tables))
    except (KB.KvBitsRefused, ValueError) as e:
        raise SystemExit(f"KV bit ceilings: {e}") from None
    args.kv_layer_spec = plan.spec
    head = getattr(plan, "headroom_bits", None)
    print(f"[kv-bits] per-layer storage: {plan.spec}" + (f"; unspendable headroom {head}" if head else ""), file=sys.stderr)


def _draft_head_ids(spec: str, cfg: ModelConfig):
    """Token ids of the shortlist draft head named by --draft-head (None: the full head)."""
    if not spec:
        return None
    if spec.isdigit():
        n = int(spec)
        if not 8 <= n <= cfg.vocab:
            raise SystemExit(f"--draft-head: a count between 8 and the vocabulary size ({cfg.vocab})")
        return list(range(n - n % 8))
    import os
    if not os.path.exists(spec):
        raise SystemExit(f"--draft-head: {spec} is neither a count nor a file")
    if spec.endswith(".npy"):
        import numpy as np
        ids = [int(v) for v in np.load(spec).reshape(-1)]
    elif spec.endswith(".pt"):
        ids = [int(v) for v in torch.load(spec).reshape(-1)]
    else:
        with open(spec) as f:
            ids = [int(line) for line in f.read().split()]
    ids = sorted(set(ids))
    return ids[: len(ids) - len(ids) % 8]


def program_factory(args, cfg: ModelConfig, weights, kv, shard=None, comm=None):
    """Factory of the ordinary (non-speculative) Program for a KV storage plan (`kv`: one format or one per layer);
    `shard` / `comm`: this rank's geometry and communicator under tensor parallelism."""
    if str(args.device).startswith("cuda"):
        from .runtime.gpu_program import GpuProgram

        descent = None
        hot_tier, floor = 0, ""
        if getattr(args, "kv_tier_formats", ""):
            from .kv.policy import parse_tier_formats, tier_formats_on_ladder
            if kv != "mixed" and not (isinstance(kv, (list, tuple)) and "mixed" in kv):
                raise SystemExit("--kv-tier-formats shapes the per-cell tiers of --kv-dtype mixed")
            try:
                hot_tier, floor = tier_formats_on_ladder(parse_tier_formats(args.kv_tier_formats))
            except ValueError as e:
                raise SystemExit(f"--kv-tier-formats: {e}") from None
        if getattr(args, "kv_descent_age", 0) > 0:
            from .kv.descent import DescentConfig
            table = None
            if getattr(args, "kv_descent_floor_nats", 0.0) > 0:
                from .kv.descent import CellCostTable
                if getattr(args, "kv_descent_target_mib", 0.0) <= 0:
                    raise SystemExit("--kv-descent-floor-nats bounds the solve toward --kv-descent-target-mib: give the target")
                costs = [float(v) for v in str(args.kv_descent_rung_nats).split(",")]
                if len(costs) != 2 or min(costs) < 0:
                    raise SystemExit("--kv-descent-rung-nats takes two non-negative numbers: loss of a cell entering fp8, nvfp4")
                table = CellCostTable((0.0, costs[0], costs[1]), float(args.kv_descent_floor_nats), floor_measured=True)
            descent = DescentConfig(min_age_tokens=int(args.kv_descent_age), floor=floor, solve_table=table,
                                    target_resident_bytes=int(getattr(args, "kv_descent_target_mib", 0.0) * (1 << 20)))

        def factory():
            text = {k: v for k, v in weights.items() if not k.startswith("vision/")}
            prog = GpuProgram(cfg, text, args.device, descent=descent, mixed_hot_tier=hot_tier, max_lanes=args.max_lanes,
                              max_context=args.max_context,
                              kv_format=kv, page_size=args.page_size, prefill_chunk=args.prefill_chunk,
                              use_graph=not args.no_graphs, kv_pages=resolve_kv_pages(args, cfg, kv), shard=shard,
                              comm=comm, weight_budget_bytes=int(args.weight_budget_gib * (1 << 30)) if args.weight_budget_gib > 0 else None)
            load_row_scale(args, cfg, prog.model)
            prog.anchor_interval = max(0, int(getattr(args, "anchor_interval", 0)))
            prog.kv.cold_slots = bool(getattr(args, "cold_slots", False))
            apply_cold_policy(args, prog)
            if getattr(args, "planner", "lru") != "lru":
                from .runtime.planner import MaterializationPlanner
                from .utils.calib import load_preset   # built-in name or file:<path> written by utils/calib.py
                prog.planner = MaterializationPlanner(load_preset(args.planner))
            return attach_vision(args, cfg, weights, prog)
    elif getattr(args, "_package", None) is not None:
        def factory():
            from .runtime.program import PackageProgram
            prog = PackageProgram(args._package, weights, max_lanes=args.max_lanes, max_context=args.max_context)
            apply_cold_policy(args, prog)
            return prog
    else:
        def factory():
            prog = ReferenceProgram(cfg, weights, max_lanes=args.max_lanes, max_context=args.max_context,
                                    kv_format=kv if isinstance(kv, str) else "bf16")
            apply_cold_policy(args, prog)
            return attach_vision(args, cfg, weights, prog)
    return factory


def resolve_kv_pages(args, cfg: ModelConfig, kv) -> Optional[int]:
    """--kv-capacity: 'full' (every lane can reach max_context), a token count, or 'auto' (what the free device memory
    holds after the weights, less --kv-headroom-gib, along the layout's affine capacity curve)."""
    from .runtime import capacity as CAP
    spec = str(getattr(args, "kv_capacity", "full"))
    if spec == "full":
        return None
    curve = CAP.build_curve(cfg, kv, args.page_size, args.max_context, args.max_lanes)
    if spec == "auto":
        free, _ = torch.cuda.mem_get_info(torch.device(args.device))
        plan = CAP.resolve(curve, args.page_size, args.max_context, free_bytes=int(free),
                           headroom_bytes=int(args.kv_headroom_gib * (1 << 30)))
    else:
        plan = CAP.resolve(curve, args.page_size, args.max_context, explicit_tokens=int(spec))
    print(json.dumps({"kv_capacity": {"policy": plan.policy, "pages": plan.pages, "tokens": plan.tokens,
                                      "reserved_bytes": plan.reserved_bytes}}), file=sys.stderr)
    return plan.pages


def load_row_scale(args, cfg: ModelConfig, model) -> int:
    """K row-scale table from --kv-rowscale, NINFER_KV_ROWSCALE or the artifact's side file; none of them: feature off."""
    import os
    from .kv import rowscale as RS
    path = getattr(args, "kv_rowscale", None) or os.environ.get("NINFER_KV_ROWSCALE")
    if not path and getattr(args, "artifact", None) and os.path.exists(RS.side_file(args.artifact)):
        path = RS.side_file(args.artifact)
    if not path:
        return 0
    table = RS.read_table(path)
    RS.validate(table, len(cfg.attn_layers), cfg.n_kv_heads, cfg.head_dim)
    return RS.load_into(model, table, cfg.attn_layers)


def cmd_packages(args) -> int:
    """The closed package table: what each registered model needs and whether this engine serves it."""
    from .models import packages as PK
    ids = [args.model] if args.model else sorted(PK.PACKAGES)
    for mid in ids:
        print(json.dumps(PK.describe(mid)))
    return 0


def cmd_kv_rowscale(args) -> int:
    """Side-file tool: write an identity table, or validate a table against a model geometry."""
    from .kv import rowscale as RS
    cfg = get_config(args.model)
    L, H, D = len(cfg.attn_layers), cfg.n_kv_heads, cfg.head_dim
    if args.identity:
        RS.write_table(args.identity, torch.ones((L, H, D)), tag=args.tag, identity=True)
        print(json.dumps({"wrote": args.identity, "layers": L, "kv_heads": H, "head_dim": D, "identity": True}))
        return 0
    try:
        t = RS.read_table(args.validate)
        RS.validate(t, L, H, D)
    except RS.RowScaleError as e:
        print(json.dumps({"valid": False, "error": str(e)}))
        return 1
    print(json.dumps({"valid": True, "geometry": list(t.geometry), "identity": t.identity, "tag": t.tag,
                      "min": float(t.scales.float().min()), "max": float(t.scales.float().max())}))
    return 0


# ---------------------------------------------------------------------------------------------------------
def cmd_generate(args) -> int:
    from .serve.service import GenerationService, GenRequest
    if getattr(args, "kv_score_table", ""):
        from .kv import kv_bits
        return kv_bits.main(["score-table", args.kv_score_table] + (["--from", args.kv_tier_scores] if args.kv_tier_scores else []))
    if getattr(args, "capability_report", False):
        from . import hostdiag
        return hostdiag.main(["hostdiag", "cufree"])
    ranks = setup_ranks(args)
    cfg, weights, tok, name = load_model(args)
    engine = build_engine(args, cfg, weights, ranks)
    if engine is None:
        return 0     # a follower rank: it executed the leader's steps until told to stop
    svc = GenerationService(engine, tok, name)
    svc.force_greedy = bool(getattr(args, "greedy", False))
    svc.eos_ids = list(svc.eos_ids) + [int(t) for t in (getattr(args, "stop_token_id", None) or [])]
    req = GenRequest(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                     min_p=getattr(args, "min_p", None), presence_penalty=getattr(args, "presence_penalty", None),
                     frequency_penalty=getattr(args, "frequency_penalty", None),
                     seed=args.seed, enable_thinking=not args.no_think, stop=args.stop or (),
                     thinking_budget=args.thinking_budget or None)
    if getattr(args, "soft_max_tokens", 0):
        if not 1 <= args.soft_max_tokens <= args.max_tokens:
            raise SystemExit("--soft-max-tokens must lie in [1, --max-tokens]")
        req.soft_max_tokens = int(args.soft_max_tokens)
    if args.prompt_ids:
        req.prompt_ids = [int(v) for v in args.prompt_ids.split(",")]
    elif args.messages_json:
        with open(args.messages_json, encoding="utf-8") as f:
            req.messages = json.load(f)
    elif args.raw:
        req.prompt = args.prompt
    else:
        content = args.prompt
        if args.image or args.video:
            if not args.vision:
                raise SystemExit("--image / --video need --vision")
            svc.allow_media_files = True
            content = ([{"type": "image_url", "image_url": {"url": p}} for p in args.image] +
                       [{"type": "video_url", "video_url": {"url": p}} for p in args.video] +
                       [{"type": "text", "text": args.prompt}])
        req.messages = ([{"role": "system", "content": args.system}] if args.system else []) + \
                       [{"role": "user", "content": content}]
    t0 = time.perf_counter()
    result = None
    for kind, item in svc.stream(req):
        if kind == "delta":
            if item.reasoning and args.show_thinking:
                sys.stdout.write(item.reasoning)
            if item.content:
                sys.stdout.write(item.content)
            sys.stdout.flush()
        else:
            result = item
    sys.stdout.write("\n")
    dt = time.perf_counter() - t0
    stats = {"model": name, "prompt_tokens": result.prompt_tokens, "completion_tokens": result.completion_tokens,
             "finish_reason": result.finish_reason, "ttft_ms": result.ttft_ms, "total_s": round(dt, 3),
             "decode_tok_s": round((result.completion_tokens - 1) / max(1e-9, dt - (result.ttft_ms or 0) / 1e3), 2),
             "weights_bytes": total_bytes(weights)}
    if result.stop_boundary is not None:
        stats["stop_boundary"] = result.stop_boundary
    if args.print_ids:
        stats["completion_ids"] = list(result.token_ids)
    if getattr(args, "print_prompt_ids", False):
        stats["prompt_ids"] = svc.prepare(req)
    print(json.dumps(stats), file=sys.stderr)
    _shutdown(engine)
    return 0 if result.finish_reason != "error" else 1


def cmd_stage_walk(args) -> int:
    """The forward pass as a walk over pipeline stages on the CPU oracle: every stage runs its layer range, the
    residual stream crosses each boundary through a checksummed hand-off file when --stage-handoff names a directory
    (--stage-handoff-cut skips the writes: the negative control, the next stage must then refuse a missing or stale
    file).  Prints the next token and the plan; the GPU pipeline is `parallel.pp.PipelineStage` (one stage per GPU)."""
    from .models.reference_model import ReferenceModel, ReferenceSequence
    from .ops import reference as R
    from .parallel.pp import StagePlan, StagePlanError, stage_walk_reference
    args.device = "cpu"
    cfg, weights, tok, name = load_model(args)
    try:
        plan = (StagePlan.parse(args.stage_layers, cfg.n_layers) if args.stage_layers
                else StagePlan.balanced(cfg.n_layers, max(1, args.stages), cfg.full_attn_interval))
    except StagePlanError as e:
        raise SystemExit(str(e)) from None
    ids = [int(v) for v in args.prompt_ids.split(",")] if args.prompt_ids else tok.encode(args.prompt)
    model = ReferenceModel(cfg, {k: v for k, v in weights.items() if not k.startswith(("mtp/", "vision/", "dflash/"))})
    try:
        hid = stage_walk_reference(model, ReferenceSequence(cfg, R.KV_BF16), torch.tensor(ids), plan,
                                   args.stage_handoff or None, cut=bool(args.stage_handoff_cut))
    except (OSError, ValueError) as e:
        print(json.dumps({"plan": plan.spec(), "refused": str(e)}))
        return 3
    nxt = int(R.argmax_lowest(model.logits(hid[-1:]))[0])
    print(json.dumps({"model": name, "plan": plan.spec(), "stages": plan.world, "uniform": plan.uniform,
                      "handoff": args.stage_handoff or None, "prompt_tokens": len(ids), "next_token": nxt}))
    return 0


def cmd_serve(args) -> int:
    from .serve.server import serve
    from .serve.service import GenerationService
    ranks = setup_ranks(args)
    cfg, weights, tok, name = load_model(args)
    engine = build_engine(args, cfg, weights, ranks)
    if engine is None:
        return 0     # a follower rank
    timeout_s = args.queue_timeout if args.pending_timeout_ms is None else args.pending_timeout_ms / 1e3
    svc = GenerationService(engine, tok, args.served_model_name or name, max_concurrent=args.max_concurrent,
                            queue_timeout_s=timeout_s)
    engine.max_pending = max(0, int(args.max_pending_requests))
    svc.sampling_overrides = {k: getattr(args, k) for k in ("temperature", "top_p", "top_k", "min_p", "presence_penalty",
                                                            "frequency_penalty") if getattr(args, k, None) is not None}
    svc.force_greedy, svc.prefix_reuse = bool(args.greedy), not args.no_prefix_reuse
    svc.media_threads = max(1, int(args.media_preprocess_threads))
    if args.allow_remote_media:
        from .frontend import media as _media
        _media.REMOTE_FETCH["enabled"] = True
    svc.default_thinking_budget = int(args.default_thinking_budget) or None
    if args.sampling_seed is not None:
        svc.fixed_seed = int(args.sampling_seed)
    apply_retention_options(engine, args)
    relayout = None
    if args.kv_auto_relayout > 0:
        if not str(args.device).startswith("cuda") or args.spec not in ("none", "off"):
            raise SystemExit("--kv-auto-relayout needs the GPU program without speculative decoding")
        from .serve.kv_auto_relayout import KvAutoRelayout, RelayoutConfig, kv_scale_energy
        relayout = KvAutoRelayout(engine, len(cfg.attn_layers), lambda: kv_scale_energy(engine.program.kv),
                                  lambda tiers: program_factory(args, cfg, weights, list(tiers)),
                                  RelayoutConfig(target_bits=args.kv_auto_relayout, period_s=args.kv_relayout_period,
                                                 assignment=args.kv_relayout_assignment),
                                  log=lambda rec: print(json.dumps(rec), file=sys.stderr, flush=True))
        relayout.start()
    if getattr(args, "warmup", 0) > 0:
        # one short generation before the port opens: kernels are loaded, decode graphs captured, pools touched
        from .serve.service import GenRequest
        t0 = time.perf_counter()
        svc.generate(GenRequest(prompt="warm-up", max_tokens=int(args.warmup), temperature=0.0))
        print(json.dumps({"warmup_s": round(time.perf_counter() - t0, 3)}), file=sys.stderr, flush=True)
    httpd = serve(svc, args.host, args.port, args.api_key, args.request_log,
                  max_stored_responses=args.response_store_max_records,
                  max_stored_bytes=int(args.response_store_max_mib * (1 << 20)),
                  max_body_bytes=int(args.max_request_mib * (1 << 20)), cors=args.cors,
                  log_interval_s=args.log_stats_interval_ms / 1e3,
                  default_max_tokens=args.default_max_tokens or None, default_thinking=not args.no_thinking)
    print(f"ninfer-serve: {name} on http://{args.host}:{httpd.server_address[1]}", file=sys.stderr, flush=True)
    try:
        httpd.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        httpd.server_close()
        _shutdown(engine)
    return 0


def apply_retention_options(engine: Engine, args) -> None:
    """Catalogue capacities of the server's option table, applied to the engine's Program (and to every Program a
    recover() or a storage reload builds later: the factory is wrapped)."""
    def apply(prog):
        if getattr(args, "max_private_continuations", 0) > 0 and hasattr(prog, "max_checkpoints"):
            prog.max_checkpoints = int(args.max_private_continuations)
        if getattr(args, "max_shared_prefixes", 0) > 0 and hasattr(prog, "max_shared_prefixes"):
            prog.max_shared_prefixes = int(args.max_shared_prefixes)
        if getattr(args, "max_long_anchors_per_continuation", 0) > 0 and hasattr(prog, "max_anchors"):
            prog.max_anchors = int(args.max_long_anchors_per_continuation)
        if getattr(args, "host_kv_mib", 0.0) > 0 and hasattr(prog, "host_budget_bytes"):
            prog.host_budget_bytes = int(args.host_kv_mib * (1 << 20))
        return prog
    apply(engine.program)
    inner = engine._factory
    engine._factory = lambda: apply(inner())


def _shutdown(engine: Engine) -> None:
    """Stops the engine; a leader first lets the worker drain, then releases the follower ranks."""
    program = engine.program
    engine.shutdown()
    if hasattr(program, "replicated_stats"):
        program.shutdown()


def cmd_inspect(args) -> int:
    with ArtifactReader(args.path) as rd:
        print(json.dumps({"identity": {"model_id": rd.identity[0], "weights_id": rd.identity[1]},
                          "objects": [{"name": o.name, "kind": o.kind, "shape": getattr(o, "shape", None),
                                       "format": getattr(o, "format", None), "layout": getattr(o, "layout", None),
                                       "bytes": o.bytes} for o in rd.objects]}, indent=1))
    return 0


def cmd_diff(args) -> int:
    """Compares two artifacts object by object: presence, shape / format / layout, and for tensors the largest absolute
    difference of the represented values (a re-quantised artifact against its source, two conversions of one model)."""
    rows, worst = [], 0.0
    with ArtifactReader(args.a) as ra, ArtifactReader(args.b) as rb:
        names = sorted(set(ra.by_name) | set(rb.by_name))
        for n in names:
            oa, ob = ra.by_name.get(n), rb.by_name.get(n)
            if oa is None or ob is None:
                rows.append({"name": n, "status": "only_in_b" if oa is None else "only_in_a"})
                continue
            rec = {"name": n, "status": "same"}
            if oa.kind != ob.kind:
                rec["status"] = "kind_differs"
            elif oa.kind == "resource":
                if ra.resource(n) != rb.resource(n):
                    rec["status"] = "bytes_differ"
            else:
                if tuple(oa.shape) != tuple(ob.shape):
                    rec["status"] = "shape_differs"
                    rec["shapes"] = [list(oa.shape), list(ob.shape)]
                else:
                    ta, tb = ra.tensor(n).float(), rb.tensor(n).float()
                    d = float((ta - tb).abs().max()) if ta.numel() else 0.0
                    scale = float(ta.abs().max()) if ta.numel() else 0.0
                    worst = max(worst, d / scale if scale > 0 else d)
                    if oa.format != ob.format or oa.layout != ob.layout:
                        rec["status"] = "format_differs"
                        rec["formats"] = [oa.format, ob.format]
                    if d > 0:
                        rec["max_abs_diff"] = d
                        rec["relative"] = round(d / scale, 6) if scale > 0 else None
                        if rec["status"] == "same":
                            rec["status"] = "values_differ"
            if rec["status"] != "same" or args.all:
                rows.append(rec)
    for r in rows:
        print(json.dumps(r))
    print(json.dumps({"objects": len(names), "reported": len(rows), "worst_relative_diff": round(worst, 6)}))
    structural = any(r["status"] in ("only_in_a", "only_in_b", "kind_differs", "shape_differs", "bytes_differ") for r in rows)
    return 1 if structural or worst > args.tolerance else 0


def cmd_make_artifact(args) -> int:
    """Random-init artifact of a registered geometry with an embedded tokenizer and chat template."""
    cfg = get_config(args.model)
    if args.layers:
        cfg = cfg.shrink(args.layers)
    weights = random_weights(cfg, "cpu", seed=args.seed, std=0.05 if cfg.hidden <= 512 else 0.02, with_mtp=args.with_mtp)
    w = ArtifactWriter(f"{args.model}@{args.layers}" if args.layers else args.model, args.weights_id)
    for name, t in weights.items():
        leaf = name.rsplit("/", 1)[-1]
        fmt = "FP32" if t.dtype == torch.float32 else "BF16"
        if args.format != "BF16" and t.dim() == 2 and leaf in ("in_proj", "o_proj", "out_proj", "gate_up", "down", "lm_head"):
            fmt = args.format
        w.add_tensor(name, t, fmt)
    tok = Tokenizer.from_file(args.tokenizer) if args.tokenizer else Tokenizer.train_toy(
        DEFAULT_CORPUS, n_merges=min(200, max(0, cfg.vocab - 256 - len(SPECIAL_TOKENS))), added_tokens=SPECIAL_TOKENS)
    w.add_resource("tokenizer.json", tok.to_json().encode("utf-8"))
    w.add_resource("chat_template.jinja", BUILTIN_TEMPLATE.encode("utf-8"))
    w.add_resource("generation_config.json", json.dumps({"eos_token": "<|im_end|>"}).encode("utf-8"))
    w.write(args.out)
    print(f"wrote {args.out}", file=sys.stderr)
    return 0


def cmd_convert(args) -> int:
    """Hugging Face safetensors checkpoint -> .ninfer artifact (leaf by leaf, so host memory stays at one tensor),
    or the inverse with --to-hf."""
    import os
    from .convert.hf import config_from_hf, hf_to_weights, weights_to_hf
    from .convert.safetensors_io import SafetensorsSource, write_safetensors
    from .models.vision import VisionConfig
    if args.to_hf:
        with ArtifactReader(args.src) as rd:
            model_id, _ = rd.identity
            cfg = get_config(model_id)
            weights = {n: rd.tensor(n) for n in rd.tensors()}
        vision = None
        if any(k.startswith("vision/") for k in weights):
            n_blocks = 1 + max(int(k.split("/")[2]) for k in weights if k.startswith("vision/blocks/"))
            vision = VisionConfig().scaled(n_blocks, cfg.hidden)
        write_safetensors(args.out, weights_to_hf(cfg, weights, vision), {"format": "pt"})
        print(f"wrote {args.out}", file=sys.stderr)
        return 0
    is_gguf = os.path.isfile(args.src) and args.src.lower().endswith(".gguf")
    if is_gguf:
        from .convert.gguf import GgufSource, config_from_gguf
        src = GgufSource(args.src)
        cfg = get_config(args.model) if args.model else config_from_gguf(
            src.file.kv, name=os.path.splitext(os.path.basename(args.src))[0])
        if src.unmapped:
            print(f"convert: {len(src.unmapped)} GGUF tensors have no role in this family, e.g. {src.unmapped[:3]}", file=sys.stderr)
    elif args.model:
        cfg = get_config(args.model)
    else:
        with open(os.path.join(args.src, "config.json"), encoding="utf-8") as f:
            cfg = config_from_hf(json.load(f), name=os.path.basename(os.path.normpath(args.src)))
    if not is_gguf:
        src = SafetensorsSource(args.src)
    vision = None
    if args.vision or (args.vision is None and "model.visual.pos_embed.weight" in src):
        n_blocks = 1 + max(int(n.split(".")[3]) for n in src.names() if n.startswith("model.visual.blocks."))
        vision = VisionConfig().scaled(n_blocks, cfg.hidden)
    with_mtp = "mtp.fc.weight" in src and not args.no_mtp
    w = ArtifactWriter(args.model or cfg.name, args.weights_id)
    n = 0
    for name, t in hf_to_weights(cfg, src, with_mtp=with_mtp, vision=vision):
        leaf = name.rsplit("/", 1)[-1]
        fmt = "FP32" if t.dtype == torch.float32 else "BF16"
        if args.format != "BF16" and t.dim() == 2 and leaf in ("in_proj", "o_proj", "out_proj", "gate_up", "down", "lm_head") \
                and not name.startswith("vision/"):
            fmt = args.format
        w.add_tensor(name, t, fmt)
        n += 1
    for res in ("tokenizer.json", "chat_template.jinja", "generation_config.json"):
        path = os.path.join(args.src, res) if os.path.isdir(args.src) else ""
        if path and os.path.exists(path):
            with open(path, "rb") as f:
                w.add_resource(res, f.read())
    src.close()
    w.write(args.out)
    print(f"wrote {args.out}: {n} tensors, draft module {'yes' if with_mtp else 'no'}, vision {'yes' if vision else 'no'}",
          file=sys.stderr)
    return 0


def cmd_perplexity(args) -> int:
    """Corpus scoring on the oracle model: mean negative log-likelihood per token and its exponential."""
    from .models.reference_model import ReferenceModel, ReferenceSequence
    from .models.weights import dequantize_weights
    args.device = "cpu"
    cfg, weights, tok, name = load_model(args)
    with open(args.corpus, encoding="utf-8") as f:
        ids = tok.encode(f.read())[: args.max_tokens]
    if len(ids) < 2:
        raise SystemExit("corpus is too short")
    ref = ReferenceModel(cfg, dequantize_weights(weights))
    seq = ReferenceSequence(cfg)
    hidden = ref.forward(seq, torch.tensor(ids[:-1]))
    logp = torch.log_softmax(ref.logits(hidden).float(), dim=-1)
    nll = -logp[torch.arange(len(ids) - 1), torch.tensor(ids[1:])].mean().item()
    print(json.dumps({"model": name, "tokens": len(ids) - 1, "nll": round(nll, 5), "perplexity": round(math.exp(nll), 4)}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ninfer", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="one prompt -> text on stdout, stats JSON on stderr")
    add_model_args(g)
    g.add_argument("--prompt", default="Hello")
    g.add_argument("--system", default="")
    g.add_argument("--image", action="append", default=[], help="image file for the user turn (repeatable; needs --vision)")
    g.add_argument("--video", action="append", default=[], help="multi-frame image file as a video (repeatable; needs --vision)")
    g.add_argument("--raw", action="store_true", help="feed --prompt as is, without the chat template")
    g.add_argument("--prompt-ids", help="comma separated token ids")
    g.add_argument("--messages-json", help="file with an OpenAI-style messages array")
    g.add_argument("--max-tokens", type=int, default=64)
    g.add_argument("--temperature", type=float, default=None)
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--min-p", type=float, default=None)
    g.add_argument("--presence-penalty", type=float, default=None)
    g.add_argument("--frequency-penalty", type=float, default=None)
    g.add_argument("--greedy", action="store_true", help="exact arg-max whatever the sampler settings say")
    g.add_argument("--stop", action="append")
    g.add_argument("--stop-token-id", type=int, action="append", help="additional token id that ends the generation")
    g.add_argument("--print-prompt-ids", action="store_true", help="add the prompt's token ids to the stats line")
    g.add_argument("--print-token-ids", dest="print_ids", action="store_true", help="same as --print-ids")
    g.add_argument("--kv-score-table", default="", metavar="show|emit=PATH",
                   help="print or write the KV tier penalty table and exit (no model is loaded)")
    g.add_argument("--capability-report", action="store_true",
                   help="print the architecture ladder, this GPU's capability bits and the (op, format) routes, and exit")
    g.add_argument("--no-think", "--no-thinking", dest="no_think", action="store_true")
    g.add_argument("--soft-max-tokens", type=int, default=0,
                   help="from this many completion tokens on, stop at the next syntax-safe boundary (statement end, block "
                        "close, fence close, paragraph) instead of running into --max-tokens; 0 = off")
    g.add_argument("--thinking-budget", type=int, default=0,
                   help="reasoning tokens after which the reasoning frame is closed for the model (0: no cap)")
    g.add_argument("--show-thinking", action="store_true")
    g.add_argument("--print-ids", action="store_true", help="add the completion's token ids to the stats line")
    g.set_defaults(fn=cmd_generate)
    w = sub.add_parser("stage-walk", help="run the forward pass stage by stage on the CPU oracle (pipeline plan check)")
    add_model_args(w)
    w.add_argument("--stage-layers", default="", help="SPEC first-last[,first-last...] with inclusive bounds, e.g. 0-31,32-63")
    w.add_argument("--stages", type=int, default=2, help="without --stage-layers: an even split into this many stages")
    w.add_argument("--stage-handoff", default="", help="directory for the checksummed boundary files")
    w.add_argument("--stage-handoff-cut", action="store_true", help="negative control: do not write the boundary files")
    w.add_argument("--prompt", default="Hello")
    w.add_argument("--prompt-ids", default="")
    w.set_defaults(fn=cmd_stage_walk)
    s = sub.add_parser("serve", help="OpenAI / Anthropic compatible HTTP server")
    s.add_argument("--kv-auto-relayout", type=float, default=0.0,
                   help="average KV bits per element to hold: per-layer tiers follow the layers' key energy (0 = off)")
    s.add_argument("--kv-relayout-period", type=float, default=300.0, help="seconds between relayout decisions")
    s.add_argument("--kv-relayout-assignment", default="rank", choices=["rank", "knapsack"],
                   help="rank: the bit-budget allocator's tiers handed out by energy rank; knapsack: exact per-layer "
                        "choice with every layer's penalties scaled by its energy")
    add_model_args(s)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8080)
    s.add_argument("--api-key", default=None)
    s.add_argument("--served-model-name", default=None)
    s.add_argument("--max-concurrent", type=int, default=64)
    s.add_argument("--queue-timeout", type=float, default=30.0)
    s.add_argument("--request-log", "--request-log-jsonl", dest="request_log", default=None, help="JSONL request log path")
    s.add_argument("--model-id", dest="served_model_name", default=None, help="public model alias (same as --served-model-name)")
    s.add_argument("--max-pending-requests", type=int, default=256, help="requests that may wait for admission; more get 429")
    s.add_argument("--pending-timeout-ms", type=float, default=None,
                   help="longest wait for admission in milliseconds, then 503 request_queue_timeout (same as --queue-timeout in seconds)")
    s.add_argument("--log-stats-interval-ms", type=float, default=5000.0, help="throughput record interval; 0 disables it")
    s.add_argument("--max-request-mib", type=float, default=32.0, help="body-size limit before JSON parsing")
    s.add_argument("--response-store-max-records", type=int, default=512, help="locally retained Responses objects")
    s.add_argument("--response-store-max-mib", type=float, default=256.0, help="total bytes of the local Responses store")
    s.add_argument("--media-preprocess-threads", type=int, default=4, help="media decoding / resizing workers")
    s.add_argument("--default-max-tokens", type=int, default=0, help="output limit of a request that names none (0: the protocol's own default)")
    s.add_argument("--no-thinking", action="store_true", help="thinking off for requests that do not say")
    s.add_argument("--default-thinking-budget", type=int, default=0,
                   help="reasoning-token cap inherited by thinking-enabled requests that name none (0: none)")
    s.add_argument("--no-prefix-reuse", action="store_true", help="no session continuations, shared prefixes or replay frontiers")
    s.add_argument("--max-private-continuations", type=int, default=0, help="retained private frontiers (0: twice the lanes)")
    s.add_argument("--max-shared-prefixes", type=int, default=0, help="shared stable-prefix catalogue size (0: 8)")
    s.add_argument("--max-long-anchors-per-continuation", type=int, default=0, help="long anchors kept per session (0: 3)")
    s.add_argument("--host-kv-mib", type=float, default=0.0, help="pinned host budget for frontiers pushed out of the device pool")
    s.add_argument("--cors", action="store_true", help="permissive browser CORS headers")
    s.add_argument("--allow-remote-media", action="store_true",
                   help="fetch http(s):// image / video URLs of requests (size-bounded, 10 s, at most 3 redirects); off: "
                        "clients send data: URIs")
    for flag, typ in (("temperature", float), ("top-p", float), ("top-k", int), ("min-p", float),
                      ("presence-penalty", float), ("frequency-penalty", float)):
        s.add_argument(f"--{flag}", type=typ, default=None, help=f"process-level {flag} default (a request's own value wins)")
    s.add_argument("--greedy", action="store_true", help="exact arg-max for every request")
    s.add_argument("--sampling-seed", type=int, default=None, help="seed of requests that give none (default: 0)")
    s.add_argument("--warmup", type=int, default=8, help="tokens of one warm-up generation before the port opens (0 = none)")
    s.set_defaults(fn=cmd_serve)
    i = sub.add_parser("inspect", help="print an artifact's directory")
    i.add_argument("path")
    i.set_defaults(fn=cmd_inspect)
    m = sub.add_parser("make-artifact", help="write a random-init artifact with embedded frontend resources")
    m.add_argument("--model", default="tiny-dense")
    m.add_argument("--layers", type=int, default=0)
    m.add_argument("--weights-id", default="random-init-bf16")
    m.add_argument("--format", default="BF16", help="matmul weight format, e.g. BF16, NVFP4, FP8_E4M3FN_ROW_BF16S, W8G32_F16S")
    m.add_argument("--with-mtp", action="store_true")
    m.add_argument("--tokenizer")
    m.add_argument("--seed", type=int, default=0)
    m.add_argument("--out", required=True)
    m.set_defaults(fn=cmd_make_artifact)
    c = sub.add_parser("convert", help="Hugging Face safetensors checkpoint or GGUF file -> .ninfer artifact (or back with --to-hf)")
    c.add_argument("src", help="checkpoint directory / .safetensors file (or an artifact with --to-hf)")
    c.add_argument("--out", required=True)
    c.add_argument("--model", default="", help="registered geometry; default: derived from the checkpoint's config.json")
    c.add_argument("--weights-id", default="hf-import")
    c.add_argument("--format", default="BF16", help="storage format of the matmul weights in the artifact")
    c.add_argument("--vision", action=argparse.BooleanOptionalAction, default=None, help="import the vision tower (default: if present)")
    c.add_argument("--no-mtp", action="store_true", help="skip the draft module")
    c.add_argument("--to-hf", action="store_true", help="artifact -> safetensors with Hugging Face names")
    c.set_defaults(fn=cmd_convert)
    d = sub.add_parser("diff", help="compare two artifacts (objects, formats, represented values)")
    d.add_argument("a"); d.add_argument("b")
    d.add_argument("--tolerance", type=float, default=0.0, help="largest accepted relative difference of a tensor")
    d.add_argument("--all", action="store_true", help="list identical objects too")
    d.set_defaults(fn=cmd_diff)
    k = sub.add_parser("packages", help="list the registered model packages and the capability gate's verdict")
    k.add_argument("--model", default=None)
    k.set_defaults(fn=cmd_packages)
    r = sub.add_parser("kv-rowscale", help="K row-scale side file: write an identity table or validate one")
    r.add_argument("--model", default="qwen3.6-27b")
    r.add_argument("--identity", metavar="OUT", help="write an identity table for the model's geometry")
    r.add_argument("--validate", metavar="TABLE", help="check a table against the model's geometry")
    r.add_argument("--tag", default="")
    r.set_defaults(fn=cmd_kv_rowscale)
    p = sub.add_parser("perplexity", help="score a text corpus on the oracle model")
    add_model_args(p)
    p.add_argument("--corpus", required=True)
    p.add_argument("--max-tokens", type=int, default=512)
    p.set_defaults(fn=cmd_perplexity)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
