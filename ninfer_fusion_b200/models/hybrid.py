"""Hybrid GDN / gated-GQA decoder forward pass on the native kernels.

The math is the reference's layer schedule
(src/targets/qwen3_6/impl/runtime/text_context_impl.h: attn_mix :1283-1468,
gdn_mix :1470-1607, mlp_tail :1609-1618, run_layers :1830-2031) but the
structure is B200-first: one ragged token batch per step (prefill chunks and
decode rows use the same kernels), every GEMM is the tcgen05 weight-stationary
kernel with a fused epilogue, the residual add + split-K reduction + next
RMSNorm is one row kernel, and all buffers are preallocated so a decode step
can be captured once in a CUDA graph.
"""
from __future__ import annotations

import os

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .._lib import StatusWord, load_native
from ..ops.reference import rope_inv_freq, rope_inv_freq_yarn
from ..runtime.kv_cache import GdnStatePool, PagedKvCache
from .config import ModelConfig

EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU, EPI_PARTIAL = 0, 1, 2, 3
MAX_SPLITS = 8


@dataclass
class StepBatch:
    """Device-side description of one ragged step (all int32)."""
    ids: torch.Tensor          # [T]
    token_seq: torch.Tensor    # [T] sequence index inside this step (row of cu_seqlens / state_slot)
    table_row: torch.Tensor    # [T] row of the KV block table for each token
    cache_pos: torch.Tensor    # [T] position in the sequence's KV cache
    rope_pos: torch.Tensor     # [T] or [T, 3]
    kv_len: torch.Tensor       # [T] visible keys per token (cache_pos + 1)
    cu_seqlens: torch.Tensor   # [B + 1]
    state_slot: torch.Tensor   # [B] GDN state slot per sequence
    logit_rows: torch.Tensor   # [R] token indices whose logits are needed
    max_kv_len: int            # host copy, picks the attention split geometry
    n_tokens: int
    n_seqs: int
    one_token_per_seq: bool = False
    qblk_start: Optional[torch.Tensor] = None   # [NB] first token of each attention query block
    qblk_count: Optional[torch.Tensor] = None   # [NB] tokens per query block
    # draft-tree verification (all optional): per token, the parent's token index (-1 = root of its window), whether
    # the token extends the state it saw (0 = side branch), the visibility bit mask over the window's cache
    # positions and the window's first cache position
    tree_parent: Optional[torch.Tensor] = None  # int32 [T]
    tree_commit: Optional[torch.Tensor] = None  # uint8 [T]
    tree_mask: Optional[torch.Tensor] = None    # int64 [T]
    tree_base: Optional[torch.Tensor] = None    # int32 [T]
    # multimodal prefill: rows of the step whose embedding is replaced by a vision-tower output row
    embed_rows: Optional[torch.Tensor] = None   # int64 [V]
    embed_vals: Optional[torch.Tensor] = None   # bf16 [V, hidden]


class Workspace:
    """Activation buffers for up to `max_tokens` tokens; addresses are stable across steps."""

    def __init__(self, cfg: ModelConfig, max_tokens: int, max_logit_rows: int, device, max_splits_attn: int = 64,
                 shard: Optional["ShardGeometry"] = None, x_buffer: Optional[torch.Tensor] = None):
        g = shard or ShardGeometry.full(cfg)
        bf, dev = torch.bfloat16, device
        T, h = max_tokens, cfg.hidden
        self.max_tokens = T
        # residual stream; under tensor parallelism it lives in the symmetric buffer peers store into
        self.x = x_buffer if x_buffer is not None else torch.empty((T, h), dtype=bf, device=dev)
        if self.x.shape[0] < T or self.x.shape[1] != h:
            raise ValueError("residual buffer is too small for the workspace")
        self.normed = torch.empty((T, h), dtype=bf, device=dev)
        # rows are read with 16-byte vector loads: keep the leading dimension a multiple of 64 elements
        wide = (max(g.attn_in_dim, g.gdn_in_dim) + 63) // 64 * 64
        self.proj = torch.empty((T, wide), dtype=bf, device=dev)
        self.q = torch.empty((T, g.n_q_heads * cfg.head_dim), dtype=bf, device=dev)
        self.mix_attn = torch.empty((T, g.n_q_heads * cfg.head_dim), dtype=bf, device=dev)
        self.mix_gdn = torch.empty((T, g.gdn_v_dim), dtype=bf, device=dev)
        self.conv = torch.empty((T, g.gdn_conv_dim), dtype=bf, device=dev)
        inter = g.ffn_inter if cfg.moe is None else max(cfg.moe.expert_inter, cfg.moe.shared_inter)
        # zero-filled and padded to a multiple of 256 columns: a block-scaled down projection whose shard width is
        # not a multiple of its 256-value k-block reads the zero tail
        self.act = torch.zeros((T, (max(inter, 8) + 255) // 256 * 256), dtype=bf, device=dev)
        self.delta = torch.empty((T, h), dtype=bf, device=dev)
        self.partial = torch.empty((MAX_SPLITS * min(T, 256) * h,), dtype=torch.float32, device=dev)
        self.max_splits_attn = max_splits_attn
        # split-KV partials: capacity in (query token x split) rows
        self.part_rows = max(min(T, 256) * max_splits_attn, min(T, 4096))
        self.part_o = torch.empty((self.part_rows * g.n_q_heads * cfg.head_dim,), dtype=torch.float32, device=dev)
        self.part_ml = torch.empty((self.part_rows * g.n_q_heads * 2,), dtype=torch.float32, device=dev)
        self.logits = torch.empty((max_logit_rows, g.vocab_rows), dtype=bf, device=dev)
        self.head_in = torch.empty((max_logit_rows, h), dtype=bf, device=dev)
        self.next_ids = torch.empty((max_logit_rows,), dtype=torch.int32, device=dev)
        self._mtp = None
        self._dev = dev

    def mtp_scratch(self):
        """[3, max_tokens, hidden] bf16 scratch of the draft module (embedding, two normalised inputs), made on first use."""
        if self._mtp is None:
            self._mtp = torch.empty((3, self.max_tokens, self.x.shape[1]), dtype=torch.bfloat16, device=self._dev)
        return self._mtp


@dataclass
class ShardGeometry:
    """Per-rank sizes of a tensor-parallel shard (world 1 = the whole model)."""
    world: int
    rank: int
    n_q_heads: int
    n_kv_heads: int
    gdn_qk_heads: int
    gdn_v_heads: int
    ffn_inter: int
    vocab_rows: int
    head_dim: int
    gdn_head_dim: int

    @staticmethod
    def full(cfg: ModelConfig) -> "ShardGeometry":
        return ShardGeometry(1, 0, cfg.n_q_heads, cfg.n_kv_heads, cfg.gdn_qk_heads, cfg.gdn_v_heads, cfg.ffn_inter,
                             cfg.vocab, cfg.head_dim, cfg.gdn_head_dim)

    @property
    def attn_in_dim(self) -> int:
        return (2 * self.n_q_heads + 2 * self.n_kv_heads) * self.head_dim

    @property
    def gdn_qk_dim(self) -> int:
        return self.gdn_qk_heads * self.gdn_head_dim

    @property
    def gdn_v_dim(self) -> int:
        return self.gdn_v_heads * self.gdn_head_dim

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_qk_dim + self.gdn_v_dim

    @property
    def gdn_in_dim(self) -> int:
        return self.gdn_conv_dim + self.gdn_v_dim + 2 * self.gdn_v_heads


def pick_attention_split(max_kv_len: int, n_work: int, sm_count: int = 148, max_splits: int = 64,
                         waves: int = 2) -> tuple[int, int]:
    """Keys per split (multiple of 128) and split count for `n_work` (query, kv-head) items.

    Aim for about `waves` items per SM: two for the kernels that run one CTA per item, eight for the persistent
    tcgen05 kernel (its CTAs walk a list of items, so many small items balance better than few large ones).  The
    split size only depends on the context bucket, so decode and verify of the same position use the same ranges."""
    bucket = 128
    while bucket < max_kv_len:
        bucket *= 2
    want = max(1, (waves * sm_count + n_work - 1) // n_work)
    split = max(128, bucket // want)
    split = 1 << (split.bit_length() - 1)          # power of two >= 128
    while (bucket + split - 1) // split > max_splits:
        split *= 2
    n_splits = (max_kv_len + split - 1) // split
    return split, max(1, n_splits)


class LaunchCounter:
    """Proxy over torch.ops.nfb200 that counts the CUDA kernels each call launches."""

    KERNELS = {"paged_attention": 2}

    def __init__(self, ops):
        self._ops = ops
        self.count = 0
        self.launches_last_forward = 0
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._ops, name)
            if name in ("gemm_pick_splits", "prefill_attn_block_tokens", "packed_attention_tile"):
                fn = raw
            elif name == "causal_conv1d_silu":
                def fn(*a, _raw=raw):
                    self.count += 2 if (a[9] and not a[10]) else 1  # + history roll unless the decode fast path
                    return _raw(*a)
            else:
                k = self.KERNELS.get(name, 1)

                def fn(*a, _raw=raw, _k=k):
                    self.count += _k
                    return _raw(*a)
            self._cache[name] = fn
        return fn


from ..ops.groupint import GroupIntWeight  # noqa: E402  (encoded Q4/Q5/Q6/W8 weight, streamed as stored)


class QuantWeight:
    """A matmul weight held as quantised planes (ops.quant): fp8 row-scale or nvfp4 block-scaled."""
    __slots__ = ("qtype", "codes", "scale", "divisor", "shape")

    def __init__(self, qtype: int, codes: torch.Tensor, scale: torch.Tensor, divisor: float, shape):
        self.qtype, self.codes, self.scale, self.divisor, self.shape = qtype, codes, scale, float(divisor), tuple(shape)

    def nbytes(self) -> int:
        return self.codes.numel() + self.scale.numel() * self.scale.element_size()


class GdnRecords:
    """Per-layer projection and convolution outputs of a verify pass, kept so that the accepted prefix can be
    replayed into the recurrent state and the conv history without recomputing the projections
    (the reference's replay records: include/ninfer/ops/gdn_replay.h:13-49, src/core/gdn_replay_records.h)."""

    def __init__(self, cfg: ModelConfig, max_tokens: int, device, shard: Optional[ShardGeometry] = None):
        g = shard or ShardGeometry.full(cfg)
        wide = (g.gdn_in_dim + 63) // 64 * 64
        n = len(cfg.gdn_layers)
        self.max_tokens = max_tokens
        self.proj = torch.empty((n, max_tokens, wide), dtype=torch.bfloat16, device=device)
        self.conv = torch.empty((n, max_tokens, g.gdn_conv_dim), dtype=torch.bfloat16, device=device)


class HybridModel:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], device, pdl: bool = False,
                 shard: Optional[ShardGeometry] = None, prefix: str = "text", ep_rank: int = 0, ep_world: int = 1,
                 ep_group=None):
        self.cfg = cfg
        self.w = weights
        self.device = torch.device(device)
        self._raw_ops = load_native()
        self.ops = LaunchCounter(self._raw_ops)
        self.gdn_chunked = os.environ.get("NFB_GDN_CHUNKED", "1") != "0"   # chunked tensor-core GDN for long prefill chunks
        self._gdn_ws = None
        self.status = StatusWord(self.device)
        self.pdl = pdl
        self.g = shard or ShardGeometry.full(cfg)
        self.prefix = prefix
        self.rope_factor = 1.0
        if cfg.rope_yarn_factor > 1.0:
            inv, self.rope_factor = rope_inv_freq_yarn(cfg.rot_dim, cfg.rope_theta, cfg.rope_yarn_factor, cfg.max_context)
            self.inv_freq = inv.to(self.device)
        else:
            self.inv_freq = rope_inv_freq(cfg.rot_dim, cfg.rope_theta).to(self.device)
        self.sm_scale = 1.0 / math.sqrt(cfg.head_dim)
        # per-layer K row-scale tables ([n_kv_heads, head_dim] bf16), set by load_k_row_scale (kv/rowscale.py)
        self.k_row_scale: Dict[int, torch.Tensor] = {}
        self._rot_scratch: Dict[tuple, torch.Tensor] = {}   # rotated activations / gate-up rows of groupwise-int weights
        self.groupint_dense_prefill = os.environ.get("NFB_GROUPINT_DENSE", "1") != "0"
        self.cluster_splitk = True  # False: split-K through an fp32 workspace + reduce kernel
        # GDN decode conv inside the in_proj epilogue (NFB_FUSE_CONV=1): one launch less per GDN layer, but the taps
        # and the history roll then sit on the critical path of the projection's leader CTAs; measured slower than
        # the separate conv kernel both on one GPU (13.78 vs 13.56 ms per round) and on a 1/8 shard (4.73 vs 4.37 ms),
        # so it is off unless asked for.
        self._fuse_conv_env = os.environ.get("NFB_FUSE_CONV")
        # decode convolution inside the recurrent GDN step (NFB_FUSE_GDN_CONV=1 switches it on)
        self._fuse_gdn_conv = os.environ.get("NFB_FUSE_GDN_CONV", "0") == "1"
        # decode: every GEMM asks L2 for the head of the NEXT GEMM's weights once its own loads are in flight
        # (NFB_L2_PREFETCH=0 switches the hint off)
        self.l2_prefetch = os.environ.get("NFB_L2_PREFETCH", "1") != "0"
        self.attn_impl = 0  # 0 = pick, 1 = SIMT, 2 = tensor-core split-KV attention
        # Feature taps for a draft model that conditions on intermediate target states (DFlash): {layer: column
        # block}; after that layer's MLP the residual stream of the step's tokens is copied into
        # feature_buf[:, block * hidden : (block + 1) * hidden].  None: nothing is copied.
        self.layer_window: Dict[int, int] = {}   # layer -> sliding window of its decode-style attention (absent: all keys)
        self.feature_taps: Optional[Dict[int, int]] = None
        self.feature_buf: Optional[torch.Tensor] = None
        self.comm = None  # tensor-parallel communicator (parallel.tp), None on one GPU
        # (norm weight, normed buffer, T) while the residual stream of the last row-parallel GEMM is still being
        # gathered from the owner ranks and ws.normed has not been written (tensor parallel, decode sizes)
        self._gathered = None
        self.act_nvfp4 = any(isinstance(t, QuantWeight) and t.qtype == 2 for t in weights.values())
        # nvfp4: producers quantise their own output for the next GEMM (NFB_FUSE_ACT_QUANT=0: stand-alone quantiser)
        self._fuse_act_quant = os.environ.get("NFB_FUSE_ACT_QUANT", "1") != "0"
        self._prequant = None
        self._qbuf: Dict[int, tuple] = {}
        self._padbuf: Dict[int, torch.Tensor] = {}
        self._qkeep: List[tuple] = []
        self.moe = None   # models.moe.MoeBlock, created with the first workspace that runs a MoE layer
        self.ep = (ep_rank, ep_world, ep_group)  # expert parallelism: experts split, the rest data-parallel
        self.expert_format = "bf16"   # "fp8_block": routed experts as e4m3 with 128 x 128 block scales
        self.moe_global_tokens: Optional[int] = None  # bound on the tokens of all ranks in a step (default world * T)
        # layer index -> index among attention / GDN layers
        self._attn_idx = {l: i for i, l in enumerate(cfg.attn_layers)}
        self._gdn_idx = {l: i for i, l in enumerate(cfg.gdn_layers)}

    # ------------------------------------------------------------------ GEMM helpers
    def _quant_scratch(self, T: int, K: int):
        """Activation code / scale buffers for a quantised GEMM with K input features (grown on demand; earlier
        buffers stay alive because captured graphs may still point at them)."""
        cur = self._qbuf.get(K)
        if cur is None or cur[0] < T:
            cap = max(T, 64 if cur is None else 2 * cur[0])
            dev = self.device
            cur = (cap, torch.empty(cap * K, dtype=torch.uint8, device=dev),
                   torch.empty(cap, dtype=torch.float32, device=dev),
                   torch.zeros(int(self.ops.nvfp4_act_scale_bytes(cap, K)) if K % 64 == 0 else 16, dtype=torch.uint8, device=dev))
            self._qkeep.append(cur)
            self._qbuf[K] = cur
        return cur

    def _add_rmsnorm(self, partial, splits, delta, resid_in, resid_out, norm_w, normed, T, N):
        """resid_out = resid_in + delta + sum(partial); normed = rmsnorm(resid_out) * (1 + norm_w).  With nvfp4
        weights the decode-sized kernel also emits the block-scaled copy of `normed` that the next GEMM consumes."""
        eps = self.cfg.rms_eps
        if self.act_nvfp4 and normed is not None and N % 256 == 0:
            _, codes, _, plane = self._quant_scratch(T, N)
            self.ops.add_rmsnorm(partial, splits, delta, resid_in, resid_out, norm_w, normed, T, N, eps, True, self.pdl,
                                 codes[: T * N // 2], plane)
            self._prequant = (normed.data_ptr(), T, N)
            return
        self.ops.add_rmsnorm(partial, splits, delta, resid_in, resid_out, norm_w, normed, T, N, eps, True, self.pdl)

    def _pad_k(self, x, K: int):
        """Activation widened with zero columns to a weight whose K was padded to the kernel's k-block."""
        if x.shape[1] == K:
            return x
        buf = self._padbuf.get(K)
        if buf is None or buf.shape[0] < x.shape[0]:
            buf = torch.zeros((max(64, 2 * x.shape[0]), K), dtype=x.dtype, device=x.device)
            self._qkeep.append(buf)
            self._padbuf[K] = buf
        out = buf[: x.shape[0]]
        out[:, : x.shape[1]].copy_(x)
        return out

    def _gemm_quant(self, x, w: QuantWeight, out, epi, resid):
        x = self._pad_k(x, w.shape[1])
        T, (N, K) = x.shape[0], w.shape
        _, codes, scale, plane = self._quant_scratch(T, K)
        splits = 1
        if self.cluster_splitk:
            kb_equiv = (K // 2 if w.qtype == 2 else K) // 2   # so that K/64 equals the kernel's 128-byte k-blocks
            splits = int(self.ops.gemm_pick_splits(T, N, kb_equiv, EPI_STORE if epi == EPI_SWIGLU else epi))
        if w.qtype == 2:
            xc = codes[: T * K // 2].view(T, K // 2)
            if self._prequant != (x.data_ptr(), T, K):
                self.ops.quant_act_nvfp4(x, xc, plane, self.pdl)
            self._prequant = None
            nxt = (None, None)
            if epi == EPI_SWIGLU and T <= 128 and (N // 2) % 64 == 0 and self._fuse_act_quant:
                # the SwiGLU epilogue also writes the activation as the down projection's W4A4 operand
                K2 = N // 2
                _, codes2, _, plane2 = self._quant_scratch(T, K2)
                nxt = (codes2[: T * K2 // 2], plane2)
            self.ops.gemm_quant(2, xc, plane, w.codes, w.scale, w.divisor, out, epi, resid, splits, self.status.tensor, self.pdl,
                                *nxt)
            if nxt[0] is not None:
                self._prequant = (out.data_ptr(), T, N // 2)
        else:
            xc = codes[: T * K].view(T, K)
            self.ops.quant_act_fp8(x, xc, scale, self.pdl)
            self.ops.gemm_quant(1, xc, scale, w.codes, w.scale, 1.0, out, epi, resid, splits, self.status.tensor, self.pdl)

    def _next_operand(self, T: int, w_next, width: int):
        """(codes, scale plane) of the nvfp4 operand a producer should write for the GEMM over `w_next`, or (None, None):
        decode sizes, W4A4 weights, no K padding."""
        if (self._fuse_act_quant and T <= 128 and isinstance(w_next, QuantWeight) and w_next.qtype == 2
                and w_next.shape[1] == width and width % 64 == 0):
            _, codes, _, plane = self._quant_scratch(T, width)
            return codes[: T * width // 2], plane
        return None, None

    def _pf(self, T: int, w_next):
        """The tensor a decode-sized GEMM should prefetch towards L2, or None."""
        if self.l2_prefetch and T <= 64 and isinstance(w_next, torch.Tensor) and w_next.is_cuda and w_next.is_contiguous():
            return w_next
        return None

    def _gemm(self, x, w, out, epi=EPI_STORE, resid=None, conv=None, prefetch=None):
        if conv is not None and not (isinstance(w, torch.Tensor) and epi == EPI_STORE):
            raise ValueError("the conv epilogue exists for bf16 weights with the store epilogue only")
        if isinstance(w, QuantWeight):
            self._gemm_quant(x, w, out, epi, resid)
            return
        if isinstance(w, GroupIntWeight):
            # Groupwise-int codes are streamed as stored for decode-sized token counts (in-register dequant).  Prefill
            # chunks take the tcgen05 GEMM on a bf16 copy decoded once, unless NFB_GROUPINT_DENSE=0 asks for the codes
            # only (no second copy of the weights; the kernel then re-reads them once per 32 tokens).
            T = x.shape[0]
            if w.usable_by_kernel() and (T <= 32 or not self.groupint_dense_prefill):
                if w.rot_block:   # codes hold W H: rotate the activations the same way (ops/rotation.py)
                    key = (T, x.shape[1])
                    if key not in self._rot_scratch:
                        self._rot_scratch[key] = torch.empty((T, x.shape[1]), dtype=x.dtype, device=x.device)
                    self.ops.hadamard_blocks(x, self._rot_scratch[key], w.rot_block)
                    x = self._rot_scratch[key]
                if epi == EPI_SWIGLU:
                    # [gate; up] rows in one pass over the codes, then silu(gate) * up in fp32
                    key = ("gu", T, w.shape[0])
                    if key not in self._rot_scratch:
                        self._rot_scratch[key] = torch.empty((T, w.shape[0]), dtype=x.dtype, device=x.device)
                    gu = self._rot_scratch[key]
                    self.ops.groupint_linear(x, w.payload, w.fmt_id, w.shape[0], w.shape[1], gu, None, self.status.tensor)
                    inter = w.shape[0] // 2
                    out.copy_(torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float())
                    return
                if epi in (EPI_STORE, EPI_RESIDUAL):
                    self.ops.groupint_linear(x, w.payload, w.fmt_id, w.shape[0], w.shape[1], out,
                                             resid if epi == EPI_RESIDUAL else None, self.status.tensor)
                    return
            w = w.dense()
        # in-cluster split-K when the output tiles alone cannot fill the GPU (decode, sharded weights)
        splits = int(self.ops.gemm_pick_splits(x.shape[0], w.shape[0], w.shape[1], epi)) if self.cluster_splitk else 1
        self.ops.gemm_bf16(x, w, out, epi, resid, None, None, splits, self.status.tensor, self.pdl, 0,
                           *(conv or (None, None, None, None)), self._pf(x.shape[0], prefetch))

    def _materialize_normed(self, ws: Workspace) -> None:
        """Writes the normalised copy that a pending gather (see `_gathered`) has left out."""
        if self._gathered is not None:
            norm_w, normed_out, T = self._gathered
            self._gathered = None
            self.comm.gather_norm(self, ws, T, norm_w, normed_out)

    def _gemm_normed(self, ws: Workspace, T: int, w, out, epi=EPI_STORE, conv=None, prefetch=None):
        """out = epilogue(normed residual @ w^T): the consumer of the last `_gemm_to_residual`.  `conv` (bf16
        weights only) fuses the decode conv + SiLU + history roll of the leading output columns into the epilogue."""
        if self._gathered is not None:
            if self.comm.can_gather(w):
                self.comm.gemm_gathered(self, ws, T, w, out, epi, conv, self._pf(T, prefetch))
                return
            self._materialize_normed(ws)
        self._gemm(ws.normed[:T], w, out, epi, conv=conv, prefetch=prefetch)

    def _gemm_to_residual(self, ws: Workspace, a, w, T: int, norm_w, normed_out, prefetch=None):
        """x += a @ w^T ; normed_out = rmsnorm(x) * (1 + norm_w).  x is ws.x[:T] (in place)."""
        cfg, ops = self.cfg, self.ops
        x = ws.x[:T]
        N, K = w.shape
        if self.comm is not None:
            # row-parallel: partial sums live on every rank; the communicator reduces them
            self.comm.gemm_reduce_residual(self, ws, a, w, T, norm_w, normed_out, self._pf(T, prefetch))
            return
        if self.cluster_splitk:
            # split-K inside a thread-block cluster (DSMEM reduction), residual add in the epilogue
            self._gemm(a, w, x, EPI_RESIDUAL, x, prefetch=prefetch)
            self._add_rmsnorm(None, 0, None, x, None, norm_w, normed_out, T, N)
            return
        splits = int(ops.gemm_pick_splits(T, N, K, EPI_PARTIAL)) if T <= 256 else 1
        if splits > 1:
            ops.gemm_bf16(a, w, None, EPI_PARTIAL, None, None, ws.partial, splits, self.status.tensor, self.pdl)
            self._add_rmsnorm(ws.partial, splits, None, x, x, norm_w, normed_out, T, N)
        else:
            ops.gemm_bf16(a, w, x, EPI_RESIDUAL, x, None, None, 1, self.status.tensor, self.pdl)
            self._add_rmsnorm(None, 0, None, x, None, norm_w, normed_out, T, N)

    # ------------------------------------------------------------------ layers
    def _attn_layer(self, ws: Workspace, b: StepBatch, kv: PagedKvCache, layer: int, T: int, prefix: str,
                    kv_index: int):
        cfg, g, ops = self.cfg, self.g, self.ops
        D = cfg.head_dim
        w_in = self.w[f"{prefix}/attn/in_proj"]
        proj = ws.proj[:T, : w_in.shape[0]]
        self._gemm_normed(ws, T, w_in, proj, prefetch=self.w[f"{prefix}/attn/o_proj"])
        q_dim, kv_dim = g.n_q_heads * D, g.n_kv_heads * D
        planes = kv.layers[kv_index]
        tiers = getattr(planes, "desc", None)   # mixed-precision layer: addresses of its tiers and of its cell map
        table = planes.block_table if getattr(planes, "block_table", None) is not None else kv.table
        q = ws.q[:T]
        ops.attn_prep(proj, 0, q_dim, q_dim + kv_dim + q_dim, g.n_q_heads, g.n_kv_heads, D,
                      self.w[f"{prefix}/attn/q_norm"], self.w[f"{prefix}/attn/k_norm"], cfg.rms_eps, True,
                      cfg.rot_dim, self.inv_freq, self.rope_factor, b.rope_pos, b.table_row, b.cache_pos, table, q,
                      planes.k_codes, planes.v_codes, planes.k_scales, planes.v_scales, kv.page_size, planes.fmt,
                      planes.group, self.pdl, planes.hadamard, self.k_row_scale.get(layer), tiers)
        gate = proj[:, q_dim + kv_dim: q_dim + kv_dim + q_dim]
        out = ws.mix_attn[:T]
        if (not b.one_token_per_seq and b.qblk_start is not None and D == 256 and self.attn_impl != 1
                and T > b.n_seqs and b.tree_mask is None):
            # prefill / wide verify: one CTA per (query block, kv head), K/V tiles dequantised once per block
            ops.paged_attention_prefill(q, g.n_q_heads, g.n_kv_heads, D, b.table_row, b.kv_len, b.qblk_start,
                                        b.qblk_count, table, planes.k_codes, planes.v_codes, planes.k_scales,
                                        planes.v_scales, kv.page_size, planes.fmt, planes.group, self.sm_scale, gate,
                                        out, self.pdl, 0, tiers)
            return out, self.w[f"{prefix}/attn/o_proj"]
        persistent = (planes.fmt == 1 and D == 256 and kv.page_size % 64 == 0 and self.attn_impl in (0, 3)
                      and os.environ.get("NFB_ATTN_TC", "1") != "0")
        split, n_splits = pick_attention_split(b.max_kv_len, T * g.n_kv_heads, max_splits=ws.max_splits_attn,
                                               waves=8 if persistent else 2)
        if persistent:
            n_splits = max(n_splits, 2)   # the kernel cuts rows at CTA boundaries: a row needs a second result slot
        chunk = max(1, ws.part_rows // n_splits)
        w_out = self.w[f"{prefix}/attn/o_proj"]
        qc, qs = self._next_operand(T, w_out, q_dim) if chunk >= T else (None, None)   # nvfp4: merge quantises its rows
        for t0 in range(0, T, chunk):
            t1 = min(T, t0 + chunk)
            ops.paged_attention(q[t0:t1], g.n_q_heads, g.n_kv_heads, D, b.table_row[t0:t1], b.kv_len[t0:t1], table,
                                planes.k_codes, planes.v_codes, planes.k_scales, planes.v_scales, kv.page_size,
                                planes.fmt, planes.group, self.sm_scale, split, n_splits, ws.part_o, ws.part_ml,
                                gate[t0:t1], out[t0:t1], None if b.tree_mask is None else b.tree_mask[t0:t1],
                                None if b.tree_base is None else b.tree_base[t0:t1], self.attn_impl, self.pdl,
                                self.layer_window.get(layer, 0), None, None, tiers, qc, qs)
        if qc is not None:
            self._prequant = (out.data_ptr(), T, q_dim)
        return out, w_out

    def _gdn_layer(self, ws: Workspace, b: StepBatch, st: GdnStatePool, layer: int, T: int, prefix: str,
                   write_state: bool = True, rec: Optional[GdnRecords] = None):
        cfg, g, ops = self.cfg, self.g, self.ops
        gi = self._gdn_idx[layer]
        w_in = self.w[f"{prefix}/gdn/in_proj"]
        # a verify pass writes its projections into the layer's record instead of the shared scratch
        proj = (ws.proj if rec is None else rec.proj[gi])[:T, : w_in.shape[0]]
        C = g.gdn_conv_dim
        conv = (ws.conv if rec is None else rec.conv[gi])[:T]
        decode = b.n_tokens == b.n_seqs and b.one_token_per_seq
        fuse_conv = self._fuse_conv_env is not None and self._fuse_conv_env != "0"
        if (fuse_conv and decode and write_state and rec is None and b.tree_parent is None and C % 128 == 0
                and isinstance(w_in, torch.Tensor) and w_in.dtype == torch.bfloat16):
            # decode: conv taps + SiLU + history roll in the projection's epilogue (token i is sequence i)
            self._gemm_normed(ws, T, w_in, proj, EPI_STORE,
                              (self.w[f"{prefix}/gdn/conv_w"], st.conv[gi], b.state_slot, conv))
        else:
            self._gemm_normed(ws, T, w_in, proj, prefetch=self.w[f"{prefix}/gdn/out_proj"])
            if (self._fuse_gdn_conv and decode and write_state and rec is None and b.tree_parent is None
                    and b.tree_commit is None):
                # decode: the four taps, SiLU and the history roll run inside the recurrent step (one launch less)
                qk = g.gdn_qk_dim
                out = ws.mix_gdn[:T]
                ops.gdn_recurrent(proj, 0, qk, 2 * qk, proj, C, C + g.gdn_v_dim, C + g.gdn_v_dim + g.gdn_v_heads,
                                  g.gdn_qk_heads, g.gdn_v_heads, self.w[f"{prefix}/gdn/A_log"],
                                  self.w[f"{prefix}/gdn/dt_bias"], self.w[f"{prefix}/gdn/norm"], cfg.rms_eps, b.cu_seqlens,
                                  b.state_slot, st.ssm[gi], True, out, self.pdl, None, None, None,
                                  self.w[f"{prefix}/gdn/conv_w"], st.conv[gi])
                return out, self.w[f"{prefix}/gdn/out_proj"]
            ops.causal_conv1d_silu(proj, 0, C, self.w[f"{prefix}/gdn/conv_w"], b.cu_seqlens, b.token_seq, b.state_slot,
                                   st.conv[gi], conv, write_state, decode, self.pdl, None, False, b.tree_parent, None)
        qk = g.gdn_qk_dim
        out = ws.mix_gdn[:T]
        # long prefill chunks take the chunked tensor-core formulation (three launches), everything else the
        # token-by-token kernels
        chunk_ws = None
        if (self.gdn_chunked and b.tree_commit is None and T >= 256 and T >= 64 * b.n_seqs and qk % 8 == 0
                and proj.stride(0) % 8 == 0 and C % 8 == 0):
            need = int(self._raw_ops.gdn_chunked_workspace_bytes(T, b.n_seqs, g.gdn_v_heads))
            if self._gdn_ws is None or self._gdn_ws.numel() < need:
                self._gdn_ws = torch.empty(need, dtype=torch.uint8, device=self.device)
            chunk_ws = self._gdn_ws
            ops.count += 2
        w_out = self.w[f"{prefix}/gdn/out_proj"]
        qc, qs = (None, None)
        if decode and chunk_ws is None and b.tree_commit is None:
            qc, qs = self._next_operand(T, w_out, g.gdn_v_dim)   # nvfp4: the step quantises its own output rows
        ops.gdn_recurrent(conv, 0, qk, 2 * qk, proj, C, C + g.gdn_v_dim, C + g.gdn_v_dim + g.gdn_v_heads,
                          g.gdn_qk_heads, g.gdn_v_heads, self.w[f"{prefix}/gdn/A_log"], self.w[f"{prefix}/gdn/dt_bias"],
                          self.w[f"{prefix}/gdn/norm"], cfg.rms_eps, b.cu_seqlens, b.state_slot, st.ssm[gi],
                          write_state, out, self.pdl, None, b.tree_commit, chunk_ws, None, None, qc, qs)
        if qc is not None:
            self._prequant = (out.data_ptr(), T, g.gdn_v_dim)
        return out, w_out

    def _mlp(self, ws: Workspace, T: int, prefix: str, next_norm_w, normed_out, next_w=None):
        w_gu = self.w[f"{prefix}/mlp/gate_up"]
        act = ws.act[:T, : w_gu.shape[0] // 2]
        w_down = self.w[f"{prefix}/mlp/down"]
        self._gemm_normed(ws, T, w_gu, act, EPI_SWIGLU, prefetch=w_down)
        self._gemm_to_residual(ws, ws.act[:T, : w_down.shape[1]], w_down, T, next_norm_w, normed_out, prefetch=next_w)

    # ------------------------------------------------------------------ forward
    def fold_gdn_tree(self, ws: Workspace, b: StepBatch, st: GdnStatePool, rec: GdnRecords, accepted: torch.Tensor,
                      last_token: torch.Tensor) -> None:
        """Tree variant of fold_gdn: `accepted` (uint8 [T]) marks the nodes of the accepted path, `last_token`
        (int32 [n_seq]) its last node.  The whole recorded window is replayed with the accepted nodes as the only
        committing tokens, so the state ends exactly after the accepted path; the conv history is rebuilt from the
        path's last three inputs."""
        cfg, g, ops = self.cfg, self.g, self.ops
        T = b.n_tokens
        C, qk = g.gdn_conv_dim, g.gdn_qk_dim
        for layer in cfg.gdn_layers:
            gi = self._gdn_idx[layer]
            p = f"{self.prefix}/layers/{layer}"
            proj = rec.proj[gi][:T, : g.gdn_in_dim]
            conv = rec.conv[gi][:T]
            ops.causal_conv1d_silu(proj, 0, C, self.w[f"{p}/gdn/conv_w"], b.cu_seqlens, b.token_seq, b.state_slot,
                                   st.conv[gi], ws.conv[:T], True, False, self.pdl, None, True, b.tree_parent, last_token)
            ops.gdn_recurrent(conv, 0, qk, 2 * qk, proj, C, C + g.gdn_v_dim, C + g.gdn_v_dim + g.gdn_v_heads,
                              g.gdn_qk_heads, g.gdn_v_heads, self.w[f"{p}/gdn/A_log"], self.w[f"{p}/gdn/dt_bias"],
                              self.w[f"{p}/gdn/norm"], cfg.rms_eps, b.cu_seqlens, b.state_slot, st.ssm[gi], True,
                              ws.mix_gdn[:T], self.pdl, None, accepted)

    def fold_gdn(self, ws: Workspace, b: StepBatch, st: GdnStatePool, rec: GdnRecords, seq_end: torch.Tensor) -> None:
        """Replays tokens [cu_seqlens[s], seq_end[s]) of the recorded verify pass `b` into the conv history and the
        recurrent state of every GDN layer (the accepted prefix of a speculative round)."""
        cfg, g, ops = self.cfg, self.g, self.ops
        T = b.n_tokens
        C, qk = g.gdn_conv_dim, g.gdn_qk_dim
        for layer in cfg.gdn_layers:
            gi = self._gdn_idx[layer]
            p = f"{self.prefix}/layers/{layer}"
            proj = rec.proj[gi][:T, : g.gdn_in_dim]
            conv = rec.conv[gi][:T]
            ops.causal_conv1d_silu(proj, 0, C, self.w[f"{p}/gdn/conv_w"], b.cu_seqlens, b.token_seq, b.state_slot,
                                   st.conv[gi], ws.conv[:T], True, False, self.pdl, seq_end, True)
            ops.gdn_recurrent(conv, 0, qk, 2 * qk, proj, C, C + g.gdn_v_dim, C + g.gdn_v_dim + g.gdn_v_heads,
                              g.gdn_qk_heads, g.gdn_v_heads, self.w[f"{p}/gdn/A_log"], self.w[f"{p}/gdn/dt_bias"],
                              self.w[f"{p}/gdn/norm"], cfg.rms_eps, b.cu_seqlens, b.state_slot, st.ssm[gi], True,
                              ws.mix_gdn[:T], self.pdl, seq_end)

    def forward_mtp(self, ws: Workspace, b: StepBatch, kv_mtp: PagedKvCache, hidden_in: torch.Tensor,
                    next_ids: torch.Tensor) -> torch.Tensor:
        """Draft module (one full-attention decoder layer sharing the embedding and the LM head): position p
        consumes the final-normed hidden state of position p and the embedding of token p + 1 and predicts
        token p + 2.  `hidden_in` [T, hidden] must not alias ws.normed.  Returns the module's final-normed
        hidden states (ws.normed[:T]), which feed the shared head and the next draft step.
        Reference: src/targets/qwen3_6/impl/runtime/mtp_impl.h, text_context_impl.h:732-1090,
        docs/maintainer/qwen3.6-35b-a3b-model.md:416-470."""
        cfg, ops, w = self.cfg, self.ops, self.w
        T, h = b.n_tokens, cfg.hidden
        scratch = ws.mtp_scratch()
        e, a_n, e_n = scratch[0, :T], scratch[1, :T], scratch[2, :T]
        ops.embed_gather(next_ids, w[f"{self.prefix}/embed"], e, self.pdl)
        self._add_rmsnorm(None, 0, None, hidden_in, None, w["mtp/pre_fc_norm_hidden"], a_n, T, h)
        self._add_rmsnorm(None, 0, None, e, None, w["mtp/pre_fc_norm_embedding"], e_n, T, h)
        fc = w["mtp/fc"]  # [hidden, 2 * hidden]: columns [hidden state ; embedding]
        x = ws.x[:T]
        self._gemm(a_n, fc[:, :h], x)
        self._gemm(e_n, fc[:, h:], x, EPI_RESIDUAL, x)
        p = "mtp/layers/0"
        self._add_rmsnorm(None, 0, None, x, None, w[f"{p}/input_norm"], ws.normed[:T], T, h)
        mix, w_out = self._attn_layer(ws, b, kv_mtp, 0, T, p, 0)
        self._gemm_to_residual(ws, mix, w_out, T, w[f"{p}/post_norm"], ws.normed[:T])
        if cfg.moe is None:
            self._mlp(ws, T, p, w["mtp/final_norm"], ws.normed[:T])
        else:
            self._materialize_normed(ws)
            if self.moe is None or self.moe.max_tokens < ws.max_tokens:
                from .moe import MoeBlock
                self.moe = MoeBlock(cfg, self.device, ws.max_tokens, *self.ep, expert_format=self.expert_format)
            self.moe.forward(self, ws, T, p, w["mtp/final_norm"], ws.normed[:T], self.moe_global_tokens)
        return ws.normed[:T]

    def forward_hidden(self, ws: Workspace, b: StepBatch, kv: PagedKvCache, st: GdnStatePool,
                       write_state: bool = True, rec: Optional[GdnRecords] = None,
                       layers: Optional[tuple] = None) -> torch.Tensor:
        """Runs all layers; returns the final-normed hidden states [T, hidden] (ws.normed).

        `layers = (first, end)` runs one pipeline stage: a stage that does not start at layer 0 finds the residual
        stream of the previous stage in ws.x[:T]; a stage that does not end at the last layer leaves its residual
        stream there (the returned tensor is then ws.x[:T])."""
        cfg, ops = self.cfg, self.ops
        T = b.n_tokens
        if T > ws.max_tokens:
            raise ValueError(f"step of {T} tokens exceeds the workspace ({ws.max_tokens})")
        first_layer, end_layer = layers if layers is not None else (0, cfg.n_layers)
        x = ws.x[:T]
        if first_layer == 0:
            ops.embed_gather(b.ids, self.w[f"{self.prefix}/embed"], x, self.pdl)
            if b.embed_rows is not None and b.embed_rows.numel():
                x.index_copy_(0, b.embed_rows, b.embed_vals)   # visual tokens replace their placeholder embeddings
        first = f"{self.prefix}/layers/{first_layer}/input_norm"
        self._add_rmsnorm(None, 0, None, x, None, self.w[first], ws.normed[:T], T, cfg.hidden)
        note_layer = getattr(self.w, "note_layer", None)   # offloaded weights rotate through a device arena
        for layer in range(first_layer, end_layer):
            p = f"{self.prefix}/layers/{layer}"
            if note_layer is not None:
                note_layer(layer)
            if cfg.is_full_attn(layer):
                mix, w_out = self._attn_layer(ws, b, kv, layer, T, p, self._attn_idx[layer])
            else:
                mix, w_out = self._gdn_layer(ws, b, st, layer, T, p, write_state, rec)
            self._gemm_to_residual(ws, mix, w_out, T, self.w[f"{p}/post_norm"], ws.normed[:T],
                                   prefetch=self.w.get(f"{p}/mlp/gate_up"))
            if layer + 1 < cfg.n_layers:
                # at a stage boundary the next layer's norm lives on the next rank, which recomputes it from the
                # residual stream: any norm weight of this rank keeps the fused kernel's shape
                nxt = self.w.get(f"{self.prefix}/layers/{layer + 1}/input_norm", self.w[f"{p}/input_norm"])
            else:
                nxt = self.w[f"{self.prefix}/final_norm"]
            if cfg.moe is None:
                if layer + 1 < cfg.n_layers:
                    kind = "attn" if cfg.is_full_attn(layer + 1) else "gdn"
                    next_w = self.w.get(f"{self.prefix}/layers/{layer + 1}/{kind}/in_proj")
                else:
                    next_w = self.w.get(f"{self.prefix}/lm_head")
                self._mlp(ws, T, p, nxt, ws.normed[:T], next_w)
            else:
                self._materialize_normed(ws)
                if self.moe is None or self.moe.max_tokens < ws.max_tokens:
                    from .moe import MoeBlock
                    self.moe = MoeBlock(cfg, self.device, ws.max_tokens, *self.ep, expert_format=self.expert_format)
                self.moe.forward(self, ws, T, p, nxt, ws.normed[:T], self.moe_global_tokens)
            if self.feature_taps is not None and layer in self.feature_taps:
                blk, h = self.feature_taps[layer], cfg.hidden
                self.feature_buf[:T, blk * h:(blk + 1) * h].copy_(ws.x[:T])
        self._materialize_normed(ws)
        return ws.normed[:T] if end_layer == cfg.n_layers else x

    def logits(self, ws: Workspace, b: StepBatch, hidden: torch.Tensor) -> torch.Tensor:
        R = b.logit_rows.numel()
        head_in = ws.head_in[:R]
        if R == hidden.shape[0]:
            head_in = hidden  # decode: every row is a logit row, in order
        else:
            torch.index_select(hidden, 0, b.logit_rows.long(), out=head_in)
        out = ws.logits[:R]
        self._gemm(head_in, self.w[f"{self.prefix}/lm_head"], out)
        return out

    def forward_greedy(self, ws: Workspace, b: StepBatch, kv: PagedKvCache, st: GdnStatePool) -> torch.Tensor:
        """One step ending in arg-max token ids for `b.logit_rows` (int32 [R], ws.next_ids)."""
        start = self.ops.count
        hidden = self.forward_hidden(ws, b, kv, st)
        if b.logit_rows.numel() == 0:
            return ws.next_ids[:0]
        lg = self.logits(ws, b, hidden)
        out = ws.next_ids[: lg.shape[0]]
        if self.comm is not None:
            self.comm.argmax(self, lg, out)
            self.ops.count += 1
        else:
            self.ops.argmax_rows(lg, out, self.pdl)
        self.ops.launches_last_forward = self.ops.count - start
        return out
