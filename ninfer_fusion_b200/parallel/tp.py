"""Tensor parallelism over one NVSwitch box: shard plan, symmetric buffers, fused collectives.

Shard rules (the reference only specifies them as host arithmetic,
src/core/shard_plan.h:56-251, docs/gfx906/TP2-SLICES.md:42-61): column-parallel
input projections (attention heads, GDN heads and the FFN intermediate are split;
a KV head is replicated when there are fewer KV heads than ranks), row-parallel
output projections, vocabulary-parallel head, replicated embedding / norms /
residual stream.  Every row-parallel GEMM is followed by a sum over ranks: here
the GEMM epilogue itself pushes its partial tiles into the owning rank over
NVLink (`gemm_bf16_push`), and one more kernel reduces, adds the residual,
all-gathers the new residual by peer stores and RMS-normalises it for the next
column-parallel GEMM (`tp_reduce_ag_norm`).  At decode sizes both hops happen
inside the GEMM (`gemm_bf16_rs_ag`: the CTA that owns a column tile waits for
the peers' tiles, reduces and pushes the new residual tile to every rank) and
the next column-parallel GEMM waits for the gathered residual in its own TMA
producer, with the RMS norm applied as a row scale in its epilogue
(`gemm_bf16_gathered`; needs `fold_norms`).  `mode="oneshot"` keeps the older
decode path (every rank receives every fp32 tile, one more kernel sums and
normalises), `mode="nccl"` a plain NCCL all-reduce as the baseline for the
same math.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .._lib import load_native
from ..models.config import ModelConfig
from ..models.hybrid import EPI_PARTIAL, MAX_SPLITS, ShardGeometry
from ..models.weights import random_weights, weight_shapes


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


def shard_geometry(cfg: ModelConfig, rank: int, world: int) -> ShardGeometry:
    if cfg.n_q_heads % world or cfg.gdn_qk_heads % world or cfg.gdn_v_heads % world:
        raise ValueError(f"head counts of {cfg.name} do not divide over {world} ranks")
    if cfg.n_kv_heads % world and world % cfg.n_kv_heads:
        raise ValueError(f"{cfg.n_kv_heads} KV heads cannot be split or replicated over {world} ranks")
    if cfg.hidden % (128 * world):
        raise ValueError(f"hidden {cfg.hidden} / {world} ranks must be a multiple of 128 (reduce-scatter tile)")
    if cfg.moe is None and (cfg.ffn_inter % (64 * world)):
        raise ValueError("FFN intermediate / world must be a multiple of 64")
    if cfg.vocab % (2 * world):
        raise ValueError("vocabulary must divide over the ranks")
    n_kv = max(1, cfg.n_kv_heads // world)
    q_l = cfg.n_q_heads // world
    if q_l % n_kv:
        raise ValueError("non-integer GQA group on a rank")
    return ShardGeometry(world, rank, q_l, n_kv, cfg.gdn_qk_heads // world, cfg.gdn_v_heads // world,
                         cfg.ffn_inter // world if cfg.moe is None else 0, cfg.vocab // world, cfg.head_dim,
                         cfg.gdn_head_dim)


def kv_head_range(cfg: ModelConfig, rank: int, world: int) -> range:
    if cfg.n_kv_heads >= world:
        per = cfg.n_kv_heads // world
        return range(rank * per, (rank + 1) * per)
    h = rank * cfg.n_kv_heads // world
    return range(h, h + 1)


def shard_weights(full: Dict[str, torch.Tensor], cfg: ModelConfig, rank: int, world: int) -> Dict[str, torch.Tensor]:
    """Slice a full weight set into rank `rank`'s shard (same names, smaller tensors)."""
    g = shard_geometry(cfg, rank, world)
    D, d = cfg.head_dim, cfg.gdn_head_dim
    out: Dict[str, torch.Tensor] = {}

    def rows(t, start, n):
        return t[start:start + n]

    q_rows = range(rank * g.n_q_heads * D, (rank + 1) * g.n_q_heads * D)
    kvh = kv_head_range(cfg, rank, world)
    for name, t in full.items():
        leaf = name.rsplit("/", 2)[-2:] if "/" in name else [name]
        key = "/".join(leaf)
        if key == "attn/in_proj":
            qd, kd = cfg.q_dim, cfg.kv_dim
            q = t[q_rows.start:q_rows.stop]
            k = t[qd + kvh.start * D: qd + kvh.stop * D]
            gate = t[qd + kd + q_rows.start: qd + kd + q_rows.stop]
            v = t[2 * qd + kd + kvh.start * D: 2 * qd + kd + kvh.stop * D]
            out[name] = torch.cat([q, k, gate, v], 0).contiguous()
        elif key == "attn/o_proj":
            out[name] = t[:, q_rows.start:q_rows.stop].contiguous()
        elif key == "gdn/in_proj":
            qk, vd, hv = cfg.gdn_qk_dim, cfg.gdn_v_dim, cfg.gdn_v_heads
            qk_l, v_l, hv_l = g.gdn_qk_dim, g.gdn_v_dim, g.gdn_v_heads
            parts = [rows(t, rank * qk_l, qk_l), rows(t, qk + rank * qk_l, qk_l),
                     rows(t, 2 * qk + rank * v_l, v_l), rows(t, 2 * qk + vd + rank * v_l, v_l),
                     rows(t, 2 * qk + 2 * vd + rank * hv_l, hv_l), rows(t, 2 * qk + 2 * vd + hv + rank * hv_l, hv_l)]
            out[name] = torch.cat(parts, 0).contiguous()
        elif key == "gdn/conv_w":
            qk, qk_l, v_l = cfg.gdn_qk_dim, g.gdn_qk_dim, g.gdn_v_dim
            out[name] = torch.cat([rows(t, rank * qk_l, qk_l), rows(t, qk + rank * qk_l, qk_l),
                                   rows(t, 2 * qk + rank * v_l, v_l)], 0).contiguous()
        elif key in ("gdn/A_log", "gdn/dt_bias"):
            out[name] = rows(t, rank * g.gdn_v_heads, g.gdn_v_heads).contiguous()
        elif key == "gdn/out_proj":
            out[name] = t[:, rank * g.gdn_v_dim:(rank + 1) * g.gdn_v_dim].contiguous()
        elif key == "mlp/gate_up":
            i, il = cfg.ffn_inter, g.ffn_inter
            out[name] = torch.cat([rows(t, rank * il, il), rows(t, i + rank * il, il)], 0).contiguous()
        elif key == "mlp/down":
            out[name] = t[:, rank * g.ffn_inter:(rank + 1) * g.ffn_inter].contiguous()
        elif name.endswith("lm_head"):
            out[name] = rows(t, rank * g.vocab_rows, g.vocab_rows).contiguous()
        else:
            out[name] = t
    return out


class TensorParallel:
    def __init__(self, cfg: ModelConfig, rank: int, world: int, device, max_tokens: int, mode: str = "fused",
                 group=None):
        self._setup(cfg, rank, world, device, max_tokens, mode, group)
        if world > 1 and dist.is_available() and dist.is_initialized():
            self.nccl_rows = int(os.environ.get("NFB_TP_NCCL_ROWS", "512"))
        self.local, handle = self.ops.symm_alloc(self.total_bytes)
        handles: List[Optional[torch.Tensor]] = [None] * world
        dist.all_gather_object(handles, handle, group=group)
        self._connect([self.local.data_ptr() if r == rank else int(self.ops.symm_open(handles[r]))
                       for r in range(world)])
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    @staticmethod
    def best_mode(world: int) -> str:
        """The faster decode mode at `world` GPUs as measured on one 8 x B200 box (27B, batch 32, ms per round, fused
        vs one-shot): 2 GPUs 8.89 / 9.60, 4 GPUs 6.67 / 6.97, 8 GPUs 6.08 / 6.44.  (Before the reduction of the
        reduce-scatter hop was spread over the grid the fused form lost at 4 and 8 GPUs: 7.56 and 8.48.)"""
        return "fused"

    @classmethod
    def loopback(cls, cfg: ModelConfig, world: int, device, max_tokens: int, mode: str = "fused") -> List["TensorParallel"]:
        """All `world` ranks inside one process on one GPU, each with its own symmetric allocation: the rank logic,
        addressing and counters of the peer-memory kernels can then be walked through phase by phase (first every
        rank's producing step, then every rank's consuming step, so that no kernel ever waits for a later launch).
        The reference exercises its rank logic on one GPU the same way (src/core/virtual_device.h:137-145)."""
        ranks = []
        for r in range(world):
            tp = cls.__new__(cls)
            tp._setup(cfg, r, world, device, max_tokens, mode, None)
            tp.local, _ = tp.ops.symm_alloc(tp.total_bytes)
            ranks.append(tp)
        bases = [tp.local.data_ptr() for tp in ranks]
        for tp in ranks:
            tp._connect(bases)
        torch.cuda.synchronize(torch.device(device))
        return ranks

    def _setup(self, cfg: ModelConfig, rank: int, world: int, device, max_tokens: int, mode: str, group) -> None:
        self.cfg, self.rank, self.world = cfg, rank, world
        self.device = torch.device(device)
        self.mode = mode
        self.group = group
        self.geometry = shard_geometry(cfg, rank, world)
        self.ops = load_native()
        self.T_cap = min(max_tokens, 4096)
        # Steps of more rows than this reduce through an NCCL all-reduce of the bf16 product instead of the push
        # protocol (fp32 tiles to the owner, reduce, all-gather): at prefill sizes the push path's two exposed hops
        # cost ~75 us per row-parallel GEMM at two GPUs (first token 76.8 ms against 67.1 ms with NCCL and 67.4 ms
        # for the same shard with no communication at all); at decode sizes the in-GEMM protocol wins.
        # (loop-back states of one process have no process group: they keep the push protocol at every size)
        self.nccl_rows = 1 << 30
        N = cfg.hidden
        self.slice = N // world
        # ---- one symmetric allocation, identical layout on every rank ----
        off = 0
        self.off: Dict[str, int] = {}
        self.one_shot_rows = min(self.T_cap, 128)   # rows handled by the decode-sized paths
        for name, nbytes in [("recv", world * self.T_cap * self.slice * 4),          # [src][T][N/W] fp32
                             ("recv_all", 2 * world * self.one_shot_rows * N * 4),   # [parity][src][rows][N] fp32
                             ("x", self.T_cap * N * 2), ("ss", 2 * self.T_cap * world * 4),
                             ("row_flag", self.T_cap * 4), ("arrival_flag", 256), ("all_flag", 256),
                             ("cand", 2 * self.T_cap * world * 8), ("argmax_flag", self.T_cap * 4),
                             # decode-sized reduce-scatter + all-gather inside the GEMM (gemm kEpiRsAg)
                             ("rs_recv", self.one_shot_rows * N * 8),       # [src][rows][N/W] (fp32 bits, epoch) pairs
                             ("rs_flag", 256),                              # (unused: the pairs carry their own flag)
                             ("rs_ss", self.one_shot_rows * 64 * 4),        # [rows][64 column tiles] fp32
                             ("x_flag", 256)]:
            self.off[name] = off
            off += _align(nbytes)
        self.total_bytes = off
        self.state = torch.zeros(int(self.ops.tp_state_bytes()), dtype=torch.uint8, device=self.device)
        self.rs_state = torch.zeros(int(self.ops.rs_state_bytes()), dtype=torch.uint8, device=self.device)
        self.fold = False   # set by fold_norms: layer norms are pure RMS scalings, their weights live in the GEMMs
        self.delta = torch.empty((self.T_cap, N), dtype=torch.bfloat16, device=self.device)

    def _connect(self, peer_bases: List[int]) -> None:
        N = self.cfg.hidden
        self.peer_bases = list(peer_bases)
        x_bytes = self.local[self.off["x"]: self.off["x"] + self.T_cap * N * 2]
        self.x = x_bytes.view(torch.bfloat16).view(self.T_cap, N)

    # ------------------------------------------------------------------ weights
    def shard(self, full: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return shard_weights(full, self.cfg, self.rank, self.world)

    def random_shard_weights(self, seed: int = 0) -> Dict[str, torch.Tensor]:
        """Random-init weights generated directly at shard shapes (replicated tensors use a shared seed)."""
        g = self.geometry
        gen_shared = torch.Generator(device=self.device).manual_seed(seed)
        gen_rank = torch.Generator(device=self.device).manual_seed(seed * 1000 + 17 + self.rank)
        cfg = self.cfg
        shapes = {
            "attn/in_proj": (g.attn_in_dim, cfg.hidden), "attn/o_proj": (cfg.hidden, g.n_q_heads * cfg.head_dim),
            "gdn/in_proj": (g.gdn_in_dim, cfg.hidden), "gdn/conv_w": (g.gdn_conv_dim, cfg.conv_kernel),
            "gdn/A_log": (g.gdn_v_heads,), "gdn/dt_bias": (g.gdn_v_heads,),
            "gdn/out_proj": (cfg.hidden, g.gdn_v_dim), "mlp/gate_up": (2 * g.ffn_inter, cfg.hidden),
            "mlp/down": (cfg.hidden, g.ffn_inter),
        }
        out = {}
        for name, shape, dt in weight_shapes(cfg):
            key = "/".join(name.rsplit("/", 2)[-2:])
            sharded = key in shapes or name.endswith("lm_head")
            shp = shapes.get(key, (g.vocab_rows, cfg.hidden) if name.endswith("lm_head") else shape)
            gen = gen_rank if sharded else gen_shared
            t = torch.empty(shp, dtype=dt, device=self.device)
            leaf = name.rsplit("/", 1)[-1]
            if leaf.endswith("norm"):
                t.normal_(0.0, 0.02, generator=gen)
                if name.endswith("gdn/norm"):
                    t.add_(1.0)
            elif leaf == "A_log":
                t.uniform_(-1.0, 1.5, generator=gen)
            elif leaf == "dt_bias":
                t.uniform_(-2.0, 1.0, generator=gen)
            elif leaf == "conv_w":
                t.normal_(0.0, 0.3, generator=gen)
            else:
                t.normal_(0.0, 0.02, generator=gen)
            out[name] = t
        return out

    def fold_norms(self, weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Moves the column weights of every layer norm that feeds a column-parallel GEMM into that GEMM
        (`W[n, k] *= 1 + norm[k]`) and zeroes the norm, so that the norm is a pure per-token scale which the
        GEMM's epilogue can apply (`gemm_bf16_gathered`).  In place; the final norm keeps its weights."""
        for name in list(weights):
            if not name.endswith(("/input_norm", "/post_norm")):
                continue
            layer = name.rsplit("/", 1)[0]
            if name.endswith("/input_norm"):
                targets = [k for k in (f"{layer}/attn/in_proj", f"{layer}/gdn/in_proj") if k in weights]
            else:
                targets = [k for k in (f"{layer}/mlp/gate_up",) if k in weights]
            if not targets:
                continue      # e.g. a MoE block: its router and experts keep the separate norm
            scale = (1.0 + weights[name].float())[None, :]
            for k in targets:
                if weights[k].dtype != torch.bfloat16 or weights[k].dim() != 2:
                    raise ValueError(f"fold_norms: {k} must still be a bf16 matrix (fold before quantising)")
                weights[k] = (weights[k].float() * scale).to(torch.bfloat16)
            weights[name] = torch.zeros_like(weights[name])
        self.fold = True
        return weights

    # ------------------------------------------------------------------ collectives
    def _rs_ag(self, model, a, w, T: int, phase: int = 0, prefetch=None) -> None:
        ops = model.ops
        splits = int(ops.gemm_pick_splits(T, w.shape[0], w.shape[1], 6))
        ops.gemm_bf16_rs_ag(a, w, splits, self.world, self.rank, self.peer_bases, self.off["rs_recv"],
                            self.off["rs_flag"], self.off["x"], self.off["rs_ss"], self.off["x_flag"],
                            self.one_shot_rows, self.cfg.hidden, self.rs_state, phase, model.status.tensor, model.pdl,
                            prefetch)

    def gather_norm(self, model, ws, T: int, norm_w, normed_out) -> None:
        """normed_out = rmsnorm(x) * (1 + norm_w) once every rank's residual tiles of the last `_rs_ag` are here."""
        model.ops.tp_gather_norm(ws.x[:T], norm_w, normed_out, self.peer_bases[self.rank], self.off["x_flag"],
                                 self.cfg.rms_eps, True, self.rs_state, model.status.tensor, model.pdl)

    def can_gather(self, w) -> bool:
        return self.fold and isinstance(w, torch.Tensor) and w.dtype == torch.bfloat16 and w.shape[1] == self.cfg.hidden

    def gemm_gathered(self, model, ws, T: int, w, out, epi: int, conv=None, prefetch=None) -> None:
        """Column-parallel GEMM straight on the gathered residual stream (waits for it, RMS norm as a row scale).
        `conv` = (conv_w, conv_state, slot per token, conv_out): decode conv + SiLU + history roll in the epilogue."""
        ops = model.ops
        splits = int(ops.gemm_pick_splits(T, w.shape[0], w.shape[1], epi))
        ops.gemm_bf16_gathered(ws.x[:T], w, out, epi, splits, self.peer_bases[self.rank], self.off["rs_ss"],
                               self.off["x_flag"], self.cfg.hidden, self.cfg.rms_eps, self.rs_state,
                               model.status.tensor, model.pdl, *(conv or (None, None, None, None)), prefetch)

    def gemm_reduce_residual(self, model, ws, a, w, T: int, norm_w, normed_out, prefetch=None) -> None:
        """x += sum_ranks(a_r @ w_r^T); normed_out = rmsnorm(x) * (1 + norm_w)."""
        cfg, ops = self.cfg, model.ops
        N = cfg.hidden
        x = ws.x[:T]
        if hasattr(w, "qtype"):
            return self._quant_reduce_residual(model, ws, a, w, T, norm_w, normed_out)
        if self.mode == "fused" and T <= self.one_shot_rows and isinstance(w, torch.Tensor):
            # decode sizes: reduce-scatter, owner-side reduction and all-gather inside the GEMM; the norm is left to
            # the consumer (a gathered GEMM when the norms are folded, else tp_gather_norm)
            self._rs_ag(model, a, w, T, prefetch=prefetch)
            if self.fold:
                model._gathered = (norm_w, normed_out, T)
            else:
                self.gather_norm(model, ws, T, norm_w, normed_out)
            return
        if self.mode == "nccl" or T > self.T_cap or T > self.nccl_rows:
            delta = self.delta[:T] if T <= self.T_cap else torch.empty((T, N), dtype=torch.bfloat16, device=self.device)
            ops.gemm_bf16(a, w, delta, 0, None, None, None, 1, model.status.tensor, model.pdl)
            dist.all_reduce(delta, group=self.group)
            ops.add_rmsnorm(None, 0, delta, x, x, norm_w, normed_out, T, N, cfg.rms_eps, True, model.pdl)
            return
        tn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256
        t_tiles = (T + tn - 1) // tn
        if T <= self.one_shot_rows:
            # decode sizes: GEMM (in-cluster split-K) pushes its fp32 tile to every rank, one kernel sums + norms
            splits = int(ops.gemm_pick_splits(T, N, w.shape[1], 5))
            arrivals = self.world * (N // 128) * t_tiles
            ops.gemm_bf16_push_all(a, w, splits, self.world, self.rank, self.peer_bases, self.off["recv_all"],
                                   self.off["all_flag"], self.one_shot_rows, self.state, model.status.tensor, model.pdl)
            ops.tp_sum_norm(self.world, self.one_shot_rows, arrivals, self.peer_bases[self.rank], self.off["recv_all"],
                            self.off["all_flag"], x, norm_w, normed_out, cfg.rms_eps, True, self.state,
                            model.status.tensor, model.pdl)
            return
        # prefill sizes: reduce-scatter by push into the owner, then reduce + all-gather + norm
        arrivals = self.world * (self.slice // 128) * t_tiles
        ops.gemm_bf16_push(a, w, 1, self.world, self.rank, self.peer_bases, self.off["recv"],
                           self.off["arrival_flag"], model.status.tensor, model.pdl)
        ops.tp_reduce_ag_norm(self.world, self.rank, T, self.T_cap, N, 1, arrivals, self.peer_bases,
                              self.off["recv"], self.off["arrival_flag"], self.off["x"], self.off["ss"],
                              self.off["row_flag"], norm_w, normed_out, cfg.rms_eps, True, self.state,
                              model.status.tensor, model.pdl)

    def _quant_reduce_residual(self, model, ws, a, w, T: int, norm_w, normed_out) -> None:
        """Row-parallel GEMM over quantised weights (fp8 / nvfp4): same peer-memory protocols, quantised operands."""
        cfg, ops = self.cfg, model.ops
        N, K = w.shape
        a = model._pad_k(a, K)
        x = ws.x[:T]
        _, codes, scale, plane = model._quant_scratch(T, K)
        if w.qtype == 2:
            xc, xs, div = codes[: T * K // 2].view(T, K // 2), plane, w.divisor
            ops.quant_act_nvfp4(a, xc, plane, model.pdl)
        else:
            xc, xs, div = codes[: T * K].view(T, K), scale, 1.0
            ops.quant_act_fp8(a, xc, scale, model.pdl)
        model._prequant = None
        if self.mode == "nccl" or T > self.T_cap or T > self.nccl_rows:
            delta = self.delta[:T] if T <= self.T_cap else torch.empty((T, N), dtype=torch.bfloat16, device=self.device)
            ops.gemm_quant(w.qtype, xc, xs, w.codes, w.scale, div, delta, 0, None, 1, model.status.tensor, model.pdl)
            dist.all_reduce(delta, group=self.group)
            ops.add_rmsnorm(None, 0, delta, x, x, norm_w, normed_out, T, N, cfg.rms_eps, True, model.pdl)
            return
        tn = 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256   # token tile of the quantised kernel
        t_tiles = (T + tn - 1) // tn
        if T <= self.one_shot_rows:
            kb_equiv = (K // 2 if w.qtype == 2 else K) // 2
            splits = int(ops.gemm_pick_splits(T, N, kb_equiv, 0))
            arrivals = self.world * (N // 128) * t_tiles
            ops.gemm_quant_push(w.qtype, xc, xs, w.codes, w.scale, div, True, splits, self.world, self.rank, self.peer_bases,
                                self.off["recv_all"], self.off["all_flag"], self.one_shot_rows, self.state,
                                model.status.tensor, model.pdl)
            ops.tp_sum_norm(self.world, self.one_shot_rows, arrivals, self.peer_bases[self.rank], self.off["recv_all"],
                            self.off["all_flag"], x, norm_w, normed_out, cfg.rms_eps, True, self.state,
                            model.status.tensor, model.pdl)
            return
        arrivals = self.world * (self.slice // 128) * t_tiles
        ops.gemm_quant_push(w.qtype, xc, xs, w.codes, w.scale, div, False, 1, self.world, self.rank, self.peer_bases,
                            self.off["recv"], self.off["arrival_flag"], self.T_cap, self.state, model.status.tensor, model.pdl)
        ops.tp_reduce_ag_norm(self.world, self.rank, T, self.T_cap, N, 1, arrivals, self.peer_bases,
                              self.off["recv"], self.off["arrival_flag"], self.off["x"], self.off["ss"],
                              self.off["row_flag"], norm_w, normed_out, cfg.rms_eps, True, self.state,
                              model.status.tensor, model.pdl)

    def argmax(self, model, logits: torch.Tensor, out: torch.Tensor) -> None:
        if self.mode == "nccl":
            local = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
            model.ops.argmax_rows(logits, local, model.pdl)
            vals = logits.float().gather(1, local.long()[:, None])[:, 0]
            allv = [torch.empty_like(vals) for _ in range(self.world)]
            alli = [torch.empty_like(local) for _ in range(self.world)]
            dist.all_gather(allv, vals, group=self.group)
            dist.all_gather(alli, local, group=self.group)
            v = torch.stack(allv, 1)
            i = torch.stack(alli, 1) + torch.arange(self.world, device=self.device, dtype=torch.int32)[None] * logits.shape[1]
            best = v.amax(1, keepdim=True)
            cand = torch.where(v == best, i, torch.full_like(i, 2 ** 31 - 1))
            out.copy_(cand.amin(1))
            return
        model.ops.tp_argmax(self.world, self.rank, self.T_cap, logits, self.peer_bases, self.off["cand"],
                            self.off["argmax_flag"], out, self.state, model.status.tensor, model.pdl)
