"""Sparse mixture-of-experts feed-forward block on the native kernels, single GPU or expert parallel.

Math (include/ninfer/ops/sparse_moe.h:36-48, docs/maintainer/qwen3.6-35b-a3b-model.md:349-386):
softmax over the routed experts -> top-k (ties: lower id) -> weights renormalised to 1;
``x += sum_j w_j * down_e(SiLU(gate_e h) * up_e h) + sigmoid(w_s h) * shared(h)``.

The reference runs this as a closed single-GPU op (router GEMV -> warp top-8 -> 9 "paths" ->
down + combine; prefill: select/scan/permute -> grouped mma.sync GEMMs).  Here the schedule is
the same on one GPU and under expert parallelism (experts split in contiguous ranges over the
ranks, attention / GDN / router / shared expert replicated and run data-parallel):

    router GEMM (tcgen05) -> moe_route -> moe_plan (histogram exchange) -> moe_push (dispatch
    all-to-all by peer stores, rows land expert-sorted) -> grouped GEMM gate_up + SwiGLU ->
    grouped GEMM down whose epilogue stores each row into the owner rank's return buffer (combine
    all-to-all fused into the GEMM) -> moe_combine (weighted sum + shared expert + residual +
    next RMSNorm).

Every cross-rank wait is bounded and reports through the model's status word.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .._lib import load_native
from .config import ModelConfig

EPI_STORE, EPI_SWIGLU = 0, 2
MOE_EPI_SWIGLU, MOE_EPI_RETURN = 0, 1


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class MoeBlock:
    """Buffers and launch sequence of the MoE block, shared by all layers of a model."""

    def __init__(self, cfg: ModelConfig, device, max_tokens: int, rank: int = 0, world: int = 1, group=None,
                 expert_format: str = "bf16"):
        if cfg.moe is None:
            raise ValueError("model has no MoE configuration")
        m = cfg.moe
        if m.n_experts % world:
            raise ValueError(f"{m.n_experts} experts do not divide over {world} ranks")
        if expert_format not in ("bf16", "fp8_block"):
            raise ValueError("expert_format must be 'bf16' or 'fp8_block'")
        if expert_format == "fp8_block" and (cfg.hidden % 128 or m.expert_inter % 128):
            raise ValueError("fp8 128x128 block-scaled experts need hidden and expert_inter in multiples of 128")
        self.expert_format = expert_format
        self.cfg, self.rank, self.world, self.group = cfg, rank, world, group
        self.device = torch.device(device)
        self.ops = load_native()
        self.max_tokens = max_tokens
        H, E, k = cfg.hidden, m.n_experts, m.top_k
        self.n_local = E // world
        self.k_per_rank = min(k, self.n_local)
        # worst case: every token of every rank sends min(k, local experts) rows to one rank
        self.cap = world * max_tokens * self.k_per_rank
        self.off: Dict[str, int] = {}
        off = 0
        for name, nbytes in [("counts", world * E * 4), ("count_flag", 256), ("recv_x", self.cap * H * 2),
                             ("recv_meta", self.cap * 4), ("arrive_flag", 256),
                             ("ret", max_tokens * k * H * 2), ("ret_flag", 256)]:
            self.off[name] = off
            off += _align(nbytes)
        self.total_bytes = off
        self.local, handle = self.ops.symm_alloc(off)
        self.peer_bases: List[int] = [self.local.data_ptr()]
        if world > 1:
            import torch.distributed as dist
            handles: List[Optional[torch.Tensor]] = [None] * world
            dist.all_gather_object(handles, handle, group=group)
            self.peer_bases = [self.local.data_ptr() if r == rank else int(self.ops.symm_open(handles[r]))
                               for r in range(world)]
        dev, i32 = self.device, torch.int32

        def view(name, nbytes, dtype):
            return self.local[self.off[name]: self.off[name] + nbytes].view(dtype)

        self.recv_x = view("recv_x", self.cap * H * 2, torch.bfloat16).view(self.cap, H)
        self.recv_meta = view("recv_meta", self.cap * 4, i32)
        self.ret = view("ret", max_tokens * k * H * 2, torch.bfloat16).view(max_tokens * k, H)
        self.hist = torch.zeros(E, dtype=i32, device=dev)
        self.ids = torch.empty((max_tokens, k), dtype=i32, device=dev)
        self.pos = torch.empty((max_tokens, k), dtype=i32, device=dev)
        self.weights = torch.empty((max_tokens, k), dtype=torch.float32, device=dev)
        self.shared_gate = torch.empty(max_tokens, dtype=torch.float32, device=dev)
        self.send_base = torch.empty(E, dtype=i32, device=dev)
        self.max_tiles_cap = self.n_local + (self.cap + 15) // 16
        self.tiles = torch.zeros((3, self.max_tiles_cap), dtype=i32, device=dev)
        self.state = torch.zeros(int(self.ops.moe_state_bytes()), dtype=torch.uint8, device=dev)
        self.act = torch.empty((self.cap, m.expert_inter), dtype=torch.bfloat16, device=dev)
        if expert_format == "fp8_block":
            u8, f32 = torch.uint8, torch.float32
            self.recv_q = torch.empty((self.cap, H), dtype=u8, device=dev)
            self.recv_qs = torch.empty((self.cap, H // 128), dtype=f32, device=dev)
            self.act_q = torch.empty((self.cap, m.expert_inter), dtype=u8, device=dev)
            self.act_qs = torch.empty((self.cap, m.expert_inter // 128), dtype=f32, device=dev)
        self.router_cols = (E + 1 + 7) // 8 * 8
        self.logits = torch.empty((max_tokens, self.router_cols), dtype=torch.bfloat16, device=dev)
        self.shared_act = torch.empty((max_tokens, m.shared_inter), dtype=torch.bfloat16, device=dev)
        self.shared_out = torch.empty((max_tokens, H), dtype=torch.bfloat16, device=dev)
        self._router: Dict[str, torch.Tensor] = {}
        self._local_experts: Dict[str, tuple] = {}
        torch.cuda.synchronize(self.device)
        if world > 1:
            import torch.distributed as dist
            dist.barrier(group=group)

    # ------------------------------------------------------------------ weights
    def _router_weight(self, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
        """Router rows [experts ; shared gate] padded with zero rows to a multiple of 8."""
        t = self._router.get(prefix)
        if t is None:
            src = w[f"{prefix}/moe/router"]
            t = torch.zeros((self.router_cols, src.shape[1]), dtype=src.dtype, device=src.device)
            t[: src.shape[0]] = src
            self._router[prefix] = t
        return t

    def _experts(self, w: Dict[str, torch.Tensor], prefix: str) -> tuple:
        """This rank's expert banks: tensors already holding only the local range are used as they are."""
        t = self._local_experts.get(prefix)
        if t is None:
            gu, dn = w[f"{prefix}/moe/experts_gate_up"], w[f"{prefix}/moe/experts_down"]
            if gu.shape[0] != self.n_local:
                lo = self.rank * self.n_local
                gu, dn = gu[lo: lo + self.n_local].contiguous(), dn[lo: lo + self.n_local].contiguous()
            t = (gu, dn)
            if self.expert_format == "fp8_block" and gu.dtype != torch.uint8:
                from ..ops import quant as Q
                t = Q.quantize_fp8_block128(gu) + Q.quantize_fp8_block128(dn)   # (gu codes, gu scales, dn codes, dn scales)
            self._local_experts[prefix] = t
        return t

    # ------------------------------------------------------------------ forward
    def forward(self, model, ws, T: int, prefix: str, next_norm_w, normed_out, global_tokens: Optional[int] = None):
        """ws.x[:T] += moe(ws.normed[:T]); normed_out = rmsnorm(ws.x[:T]) * (1 + next_norm_w).

        `global_tokens` bounds the tokens of all ranks in this step (default world * T: equal batches).
        """
        cfg, m, ops = self.cfg, self.cfg.moe, model.ops
        if T > self.max_tokens:
            raise ValueError(f"MoE step of {T} tokens exceeds the block's capacity ({self.max_tokens})")
        E, k, W = m.n_experts, m.top_k, self.world
        status = model.status.tensor
        normed = ws.normed[:T]
        logits = self.logits[:T]
        model._gemm(normed, self._router_weight(model.w, prefix), logits)
        ids, pos, wts, sgate = self.ids[:T], self.pos[:T], self.weights[:T], self.shared_gate[:T]
        ops.moe_route(logits, E, k, m.norm_topk, True, self.hist, ids, wts, pos, sgate)
        g_tokens = W * T if global_tokens is None else global_tokens
        tn = int(ops.moe_tile_tokens(g_tokens * k / E))
        if self.expert_format == "fp8_block":
            tn = min(tn, 128)   # the two-level accumulation keeps one fp32 register per token of the tile
        rows_bound = min(self.cap, g_tokens * self.k_per_rank)
        max_tiles = min(self.max_tiles_cap, self.n_local + (rows_bound + tn - 1) // tn)
        ops.moe_plan(W, self.rank, E, tn, self.cap, self.hist, self.peer_bases, self.off["counts"],
                     self.off["count_flag"], self.send_base, self.tiles, self.state, status)
        ops.moe_push(W, self.rank, E, self.cap, normed, ids, pos, self.send_base, self.peer_bases,
                     self.off["recv_x"], self.off["recv_meta"], self.off["arrive_flag"], self.state, status)
        if self.expert_format == "fp8_block":
            gu_q, gu_s, dn_q, dn_s = self._experts(model.w, prefix)
            # one CTA per row that this step can deliver here (not per row of the worst-case receive capacity, which
            # is world x max_tokens x top-k rows: 131072 CTAs that exit at once cost more than the GEMM they feed)
            rb = rows_bound
            ops.moe_quant_rows_block128(self.recv_x[:rb], self.recv_q[:rb], self.recv_qs[:rb], self.state)
            ops.moe_gemm_fp8(self.recv_q, self.recv_qs, gu_q, gu_s, MOE_EPI_SWIGLU, tn, max_tiles, self.tiles, self.state,
                             self.act, W, None, self.peer_bases, 0, 0, status)
            ops.moe_quant_rows_block128(self.act[:rb], self.act_q[:rb], self.act_qs[:rb], self.state)
            ops.moe_gemm_fp8(self.act_q, self.act_qs, dn_q, dn_s, MOE_EPI_RETURN, tn, max_tiles, self.tiles, self.state,
                             None, W, self.recv_meta, self.peer_bases, self.off["ret"], self.off["ret_flag"], status)
        else:
            gate_up, down = self._experts(model.w, prefix)
            ops.moe_gemm(self.recv_x, gate_up, MOE_EPI_SWIGLU, tn, max_tiles, self.tiles, self.state, self.act, W, None,
                         self.peer_bases, 0, 0, status)
            ops.moe_gemm(self.act, down, MOE_EPI_RETURN, tn, max_tiles, self.tiles, self.state, None, W, self.recv_meta,
                         self.peer_bases, self.off["ret"], self.off["ret_flag"], status)
        # shared expert (replicated): dense SwiGLU MLP on the local tokens
        sact, sout = self.shared_act[:T], self.shared_out[:T]
        model._gemm(normed, model.w[f"{prefix}/moe/shared_gate_up"], sact, EPI_SWIGLU)
        model._gemm(sact, model.w[f"{prefix}/moe/shared_down"], sout)
        ops.moe_combine(ws.x[:T], wts, self.ret, self.peer_bases[self.rank], self.off["ret_flag"], sout, sgate,
                        next_norm_w, normed_out, cfg.rms_eps, self.state, status)
