"""Groupwise-integer streaming linear (Q4/Q5/Q6 g64, W8 g32): kernel vs an fp32 oracle over the represented weights.

The kernel reads the artifact's encoded row-split object directly; the oracle decodes the same bytes with the numpy
decoder and multiplies in fp32.  Sums inside a group are exact integer-times-bf16 products in fp32 and the scales
are applied in fp32, so the only differences are summation order and the bf16 rounding of the output.
"""
import pytest
import torch

from ninfer_fusion_b200.ops import groupint as G

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from ninfer_fusion_b200._lib import load_native
    return load_native()


def _check(y, ref, tag):
    y = y.float().cpu()
    scale = ref.abs().max().item() + 1e-6
    err = (y - ref).abs().max().item()
    assert err <= 8e-3 * scale, f"{tag}: max abs err {err:.4g} vs range {scale:.4g}"


@pytest.mark.parametrize("fmt", ["q4", "q5", "q6", "w8"])
@pytest.mark.parametrize("T,N,K", [(1, 64, 128), (5, 208, 320), (17, 512, 1024), (32, 9600, 512), (32, 160, 2112)])
def test_linear_matches_oracle(ops, fmt, T, N, K):
    g = torch.Generator().manual_seed(1000 * T + N + K)
    w = torch.randn((N, K), generator=g) * 0.05
    w[:, ::37] *= 6.0                      # outlier columns so that group scales differ a lot
    x = torch.randn((T, K), generator=g).to(torch.bfloat16).cuda()
    gw = G.GroupIntWeight.from_dense(w, fmt, device="cuda")
    assert gw.usable_by_kernel()
    y = G.linear(ops, x, gw)
    torch.cuda.synchronize()
    _check(y, G.linear_reference(x, gw), f"{fmt} T={T} N={N} K={K}")


@pytest.mark.parametrize("fmt", ["q4", "q6", "w8"])
def test_linear_add_in_place_and_token_chunks(ops, fmt):
    T, N, K = 70, 256, 768                 # three weight passes of 32 + 32 + 6 tokens
    g = torch.Generator().manual_seed(7)
    w = torch.randn((N, K), generator=g) * 0.03
    x = torch.randn((T, K), generator=g).to(torch.bfloat16).cuda()
    resid = torch.randn((T, N), generator=g).to(torch.bfloat16).cuda()
    gw = G.GroupIntWeight.from_dense(w, fmt, device="cuda")
    ref = G.linear_reference(x, gw, resid)
    out = resid.clone()
    G.linear(ops, x, gw, out=out, resid=out)   # residual stream updated in place, as o_proj / down do
    torch.cuda.synchronize()
    _check(out, ref, f"{fmt} linear_add")


@pytest.mark.parametrize("fmt", ["q5", "w8"])
def test_linear_pair(ops, fmt):
    T, K = 9, 640
    g = torch.Generator().manual_seed(11)
    w0 = torch.randn((96, K), generator=g) * 0.05
    w1 = torch.randn((352, K), generator=g) * 0.05
    x = torch.randn((T, K), generator=g).to(torch.bfloat16).cuda()
    a, b = G.GroupIntWeight.from_dense(w0, fmt, device="cuda"), G.GroupIntWeight.from_dense(w1, fmt, device="cuda")
    y0, y1 = G.linear_pair(ops, x, a, b)
    torch.cuda.synchronize()
    _check(y0, G.linear_reference(x, a), f"{fmt} pair[0]")
    _check(y1, G.linear_reference(x, b), f"{fmt} pair[1]")


def test_refusals(ops):
    w = G.GroupIntWeight.from_dense(torch.randn(24, 128), "q4", device="cuda")     # 24 rows: not a multiple of 16
    x = torch.zeros((2, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 16"):
        G.linear(ops, x, w)
    w = G.GroupIntWeight.from_dense(torch.randn(32, 96), "q4", device="cuda")      # K = 96: not a multiple of 64
    with pytest.raises(RuntimeError, match="multiple of 64"):
        G.linear(ops, torch.zeros((2, 96), dtype=torch.bfloat16, device="cuda"), w)


def test_model_decodes_with_stored_q4_weights(ops):
    """A tiny hybrid model whose matmul weights stay Q4 codes: prefill (bf16 copy, tcgen05 GEMM) and decode
    (streaming kernel on the codes) follow the oracle run on the represented values."""
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.reference_model import ReferenceModel, ReferenceSequence
    from ninfer_fusion_b200.models.weights import dequantize_weights, quantize_weights, random_weights
    from ninfer_fusion_b200.ops import reference as R
    from ninfer_fusion_b200.runtime.generator import Generator

    cfg = TINY_DENSE
    qw = quantize_weights(random_weights(cfg, "cuda", seed=7, std=0.05), "q4")
    assert sum(isinstance(v, G.GroupIntWeight) for v in qw.values()) >= 3 * cfg.n_layers
    gen = Generator(cfg, qw, "cuda", max_batch=4, max_context=512, kv_format="bf16", page_size=16, prefill_chunk=64,
                    use_graph=False)
    ref = ReferenceModel(cfg, {k: v.cpu() for k, v in dequantize_weights(qw).items()})
    torch.manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (21, 40)]
    got = gen.generate(prompts, 5)
    agree = total = 0
    for b, p in enumerate(prompts):
        seq = ReferenceSequence(cfg, R.KV_BF16)
        h = ref.forward(seq, torch.tensor(p))
        for i in range(5):
            logits = ref.logits(h[-1:])[0]
            top2 = torch.topk(logits, 2).values
            tok = int(got[b][i])
            # follow the engine's token; count a step as checked when the oracle's choice is not a near-tie
            if (top2[0] - top2[1]).item() > 0.02 * logits.abs().max().item():
                total += 1
                agree += int(tok == int(logits.argmax()))
            h = ref.forward(seq, torch.tensor([tok]))
    assert total >= 2 and agree == total, (agree, total, got)


@pytest.mark.parametrize("block", [64, 128, 256])
def test_hadamard_blocks_kernel(ops, block):
    from ninfer_fusion_b200.ops import rotation as ROT
    g = torch.Generator().manual_seed(block)
    x = torch.randn((37, 1024), generator=g).to(torch.bfloat16).cuda()
    y = ROT.rotate(ops, x, block)
    torch.cuda.synchronize()
    ref = ROT.rotate_reference(x.cpu(), block)
    assert (y.float().cpu() - ref).abs().max() <= 2e-2 * ref.abs().max()
    wide = torch.zeros((4, 2048), dtype=torch.bfloat16, device="cuda")
    view = wide[:, :1024]                       # strided rows, in place
    view.copy_(x[:4])
    ROT.rotate(ops, view, block, out=view)
    torch.cuda.synchronize()
    assert torch.equal(view, y[:4]) and float(wide[:, 1024:].abs().max()) == 0.0
    with pytest.raises(RuntimeError, match="multiple of the block"):
        ops.hadamard_blocks(x[:, :96].contiguous(), torch.empty((37, 96), dtype=torch.bfloat16, device="cuda"), 64)


def test_rotated_q4_linear_and_model(ops):
    """Q4 codes of W H with the activations rotated on the device: the result follows the oracle of the represented
    weight, and a tiny model with '+h64' weights decodes like its oracle."""
    g = torch.Generator().manual_seed(3)
    w = torch.randn((256, 1024), generator=g) * 0.02
    w[:, ::64] *= 25.0
    x = torch.randn((9, 1024), generator=g).to(torch.bfloat16).cuda()
    gw = G.GroupIntWeight.from_dense(w, "q4", device="cuda", rot_block=64)
    y = G.linear(ops, x, gw)
    torch.cuda.synchronize()
    _check(y, G.linear_reference(x, gw), "rotated q4")
    plain = G.GroupIntWeight.from_dense(w, "q4", device="cuda")
    exact = x.float().cpu() @ w.t()
    e_rot = (y.float().cpu() - exact).pow(2).mean().sqrt()
    e_plain = (G.linear(ops, x, plain).float().cpu() - exact).pow(2).mean().sqrt()
    assert e_rot < 0.7 * e_plain

    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.reference_model import ReferenceModel, ReferenceSequence
    from ninfer_fusion_b200.models.weights import dequantize_weights, quantize_weights, random_weights
    from ninfer_fusion_b200.ops import reference as R
    from ninfer_fusion_b200.runtime.generator import Generator
    cfg = TINY_DENSE
    qw = quantize_weights(random_weights(cfg, "cuda", seed=7, std=0.05), "q4+h64")
    assert any(isinstance(v, G.GroupIntWeight) and v.rot_block == 64 for v in qw.values())
    gen = Generator(cfg, qw, "cuda", max_batch=2, max_context=256, kv_format="bf16", page_size=16, prefill_chunk=64,
                    use_graph=False)
    ref = ReferenceModel(cfg, {k: v.cpu() for k, v in dequantize_weights(qw).items()})
    torch.manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (21, 30)]
    gen.prefill(prompts)
    got = gen.ws.logits[:2].float().cpu()
    for b, p in enumerate(prompts):
        want = ref.logits(ref.forward(ReferenceSequence(cfg, R.KV_BF16), torch.tensor(p))[-1:])[0]
        assert torch.nn.functional.cosine_similarity(got[b], want, dim=0).item() > 0.995
    out = gen.generate(prompts, 4)              # decode path: rotated activations + streaming kernel
    assert all(len(o) == 4 for o in out)
    gen.model.status.check("rotated q4 decode")


def test_model_runs_on_codes_only(ops):
    """With the dense prefill copy switched off every kernel-usable weight (the SwiGLU parent included) stays codes:
    prefill streams them per 32 tokens, decode per round; logits follow the oracle of the represented weights."""
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.reference_model import ReferenceModel, ReferenceSequence
    from ninfer_fusion_b200.models.weights import dequantize_weights, quantize_weights, random_weights
    from ninfer_fusion_b200.ops import reference as R
    from ninfer_fusion_b200.runtime.generator import Generator
    cfg = TINY_DENSE
    qw = quantize_weights(random_weights(cfg, "cuda", seed=7, std=0.05), "w8")
    gen = Generator(cfg, qw, "cuda", max_batch=2, max_context=256, kv_format="bf16", page_size=16, prefill_chunk=64,
                    use_graph=False)
    gen.model.groupint_dense_prefill = False
    ref = ReferenceModel(cfg, {k: v.cpu() for k, v in dequantize_weights(qw).items()})
    torch.manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (21, 40)]   # one 61-token chunk: two weight passes
    gen.prefill(prompts)
    got = gen.ws.logits[:2].float().cpu()
    for b, p in enumerate(prompts):
        want = ref.logits(ref.forward(ReferenceSequence(cfg, R.KV_BF16), torch.tensor(p))[-1:])[0]
        assert torch.nn.functional.cosine_similarity(got[b], want, dim=0).item() > 0.995
    out = gen.generate(prompts, 4)
    assert all(len(o) == 4 for o in out)
    gen.model.status.check("codes-only run")
    usable = [v for v in qw.values() if isinstance(v, G.GroupIntWeight) and v.usable_by_kernel()]
    assert any(k.endswith("gate_up") and isinstance(v, G.GroupIntWeight) and v.usable_by_kernel() for k, v in qw.items())
    assert usable and all(v._dense is None for v in usable)
