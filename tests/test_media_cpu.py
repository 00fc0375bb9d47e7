"""Media processor and vision control on the CPU: geometry, patch packing, placeholder expansion, positions."""
import io

import numpy as np
import pytest
import torch

from ninfer_fusion_b200.frontend import media as M
from ninfer_fusion_b200.models import vision as V


def test_smart_resize_aligns_and_respects_budget():
    h, w = M.smart_resize_image(500, 333, 64 * 1024, 16 * 1024 * 1024)
    assert h % 32 == 0 and w % 32 == 0 and (h, w) == (512, 320)
    h, w = M.smart_resize_image(4000, 6000, 64 * 1024, 1024 * 1024)
    assert h % 32 == 0 and w % 32 == 0 and h * w <= 1024 * 1024
    h, w = M.smart_resize_image(40, 60, 64 * 1024, 1024 * 1024)
    assert h * w >= 64 * 1024
    with pytest.raises(ValueError):
        M.smart_resize_image(10, 4000, 1, 10 ** 9)
    h, w = M.smart_resize_video(16, 240, 320, 128 * 1024, 512 * 1024)
    assert 16 * h * w <= 512 * 1024 and h % 32 == 0


def test_pack_patches_matches_naive_loop():
    rng = np.random.default_rng(0)
    frames = rng.integers(0, 256, (2, 64, 96, 3), dtype=np.uint8)
    rows = M.pack_patches(frames)
    gh, gw = 4, 6
    assert rows.shape == (gh * gw, 1536) and rows.dtype == torch.bfloat16
    ctl = V.build_control([(1, gh, gw)])
    for r in (0, 1, 2, 3, 4, 11, 23):
        y, x = ctl.pos_yx[r]
        want = np.zeros((3, 2, 16, 16), dtype=np.float32)
        for c in range(3):
            for t in range(2):
                want[c, t] = frames[t, 16 * y:16 * y + 16, 16 * x:16 * x + 16, c] / 127.5 - 1.0
        got = rows[r].float().view(3, 2, 16, 16).numpy()
        assert np.abs(got - want).max() < 1 / 128   # bf16 rounding of values in [-1, 1]


def test_control_orders_patches_by_merge_block():
    ctl = V.build_control([(1, 4, 6), (2, 2, 2)])
    assert ctl.n_patches == 24 + 8 and ctl.n_tokens == 8
    assert ctl.segments.tolist() == [0, 24, 28, 32]
    # the first four rows are the 2x2 block at the origin
    assert ctl.pos_yx[:4].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]]
    assert ctl.pos_yx[4:8].tolist() == [[0, 2], [0, 3], [1, 2], [1, 3]]
    assert ctl.grid_hw[0].tolist() == [4, 6] and ctl.grid_hw[-1].tolist() == [2, 2]
    tiles = V.attention_tiles(ctl.segments, 16)
    assert tiles.tolist() == [[0, 0, 24], [16, 0, 24], [24, 24, 28], [28, 28, 32]]
    with pytest.raises(ValueError):
        V.build_control([(1, 3, 4)])


def test_image_item_from_png_bytes():
    from PIL import Image
    rng = np.random.default_rng(1)
    arr = rng.integers(0, 256, (70, 100, 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    proc = M.MediaProcessor(M.MediaOptions(image_min_pixels=32 * 32, image_max_pixels=256 * 256))
    item = proc.image(buf.getvalue())
    assert item.modality == "image" and item.grid == (1, 4, 6)
    assert item.patches.shape == (24, 1536) and item.n_tokens == 6
    # both frames of the temporal pair hold the same picture
    p = item.patches[0].float().view(3, 2, 16, 16)
    assert torch.equal(p[:, 0], p[:, 1])


def test_video_item_sampling_and_timestamps():
    frames = np.zeros((48, 64, 64, 3), dtype=np.uint8)
    proc = M.MediaProcessor(M.MediaOptions(video_min_pixels=1024, video_max_pixels=1 << 24, video_fps=2.0, video_min_frames=4))
    item = proc.video(frames, fps=24.0)
    assert item.modality == "video" and item.grid == (2, 4, 4) and len(item.timestamps) == 2
    assert item.timestamps[0] < item.timestamps[1] <= 47 / 24.0
    assert item.patches.shape == (2 * 16, 1536)


def test_placeholder_expansion_and_positions():
    img = M.MediaItem("image", (1, 4, 6), torch.zeros((24, 1536), dtype=torch.bfloat16))
    vid = M.MediaItem("video", (2, 2, 4), torch.zeros((16, 1536), dtype=torch.bfloat16), [0.5, 1.5])
    text = "A<|vision_start|><|image_pad|><|vision_end|>B<|vision_start|><|video_pad|><|vision_end|>C"
    out = M.expand_placeholders(text, [img, vid])
    assert out.count("<|image_pad|>") == 6 and out.count("<|video_pad|>") == 4
    assert "<0.5 seconds><|vision_start|>" in out and "<1.5 seconds>" in out
    with pytest.raises(ValueError):
        M.expand_placeholders("no media here", [img])
    IMG, VID = 900, 901
    ids = [1, 2] + [IMG] * 6 + [3] + [VID] * 2 + [4] + [VID] * 2 + [5]
    pos, delta, rows = M.build_positions(ids, [img, vid], IMG, VID)
    assert pos[:2].tolist() == [[0, 0, 0], [1, 1, 1]]
    # 2 x 3 merged grid starting at position 2
    assert pos[2:8].tolist() == [[2, 2, 2], [2, 2, 3], [2, 2, 4], [2, 3, 2], [2, 3, 3], [2, 3, 4]]
    assert pos[8].tolist() == [5, 5, 5]            # resumes after max(h, w) = 3
    assert pos[9:11].tolist() == [[6, 6, 6], [6, 6, 7]]   # 1 x 2 grid of the first temporal group
    assert pos[11].tolist() == [8, 8, 8]
    assert pos[12:14].tolist() == [[9, 9, 9], [9, 9, 10]]
    assert pos[14].tolist() == [11, 11, 11]
    assert delta == 12 - len(ids)
    assert rows.tolist() == [2, 3, 4, 5, 6, 7, 9, 10, 12, 13]
    with pytest.raises(ValueError):
        M.build_positions(ids[:-4], [img, vid], IMG, VID)


def test_vision_reference_runs_and_segments_are_independent():
    cfg = V.VisionConfig().scaled(layers=1, out_hidden=64)
    w = V.random_vision_weights(cfg, seed=3)
    torch.manual_seed(0)
    ctl_a = V.build_control([(1, 2, 2)])
    ctl_ab = V.build_control([(1, 2, 2), (1, 2, 4)])
    pa = (0.5 * torch.randn(4, cfg.patch_dim)).to(torch.bfloat16)
    pb = (0.5 * torch.randn(8, cfg.patch_dim)).to(torch.bfloat16)
    out_a = V.vision_reference(cfg, w, pa, ctl_a)
    out_ab = V.vision_reference(cfg, w, torch.cat([pa, pb]), ctl_ab)
    assert out_a.shape == (1, 64) and out_ab.shape == (3, 64)
    assert torch.allclose(out_a, out_ab[:1], atol=1e-5)   # a second item does not change the first


def test_engine_multimodal_request_on_oracle_program():
    """A chat request with an image part runs through the service, the engine and the oracle program; the image
    changes the output, a text-only engine refuses it, and a wrong prepared prompt is rejected."""
    import base64
    from PIL import Image
    from ninfer_fusion_b200 import cli
    from ninfer_fusion_b200.frontend.tokenizer import Tokenizer
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.engine import Engine, RequestError, RequestOptions
    from ninfer_fusion_b200.runtime.program import ReferenceProgram
    from ninfer_fusion_b200.serve.service import GenerationService, GenRequest

    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=3, std=0.05)
    vcfg = V.VisionConfig().scaled(layers=1, out_hidden=cfg.hidden)
    vw = V.random_vision_weights(vcfg, seed=2)
    tok = Tokenizer.train_toy(cli.DEFAULT_CORPUS, 200, cli.SPECIAL_TOKENS)
    assert tok.token_id(M.IMAGE_PAD) is not None

    def factory():
        prog = ReferenceProgram(cfg, w, max_lanes=2, max_context=512)
        prog.attach_vision(vcfg, vw)
        return prog

    engine = Engine(factory, prefill_chunk=16)
    try:
        svc = GenerationService(engine, tok, "tiny-dense:test", max_concurrent=2)
        svc.media = M.MediaProcessor(M.MediaOptions(image_min_pixels=32 * 32, image_max_pixels=64 * 64))

        def uri(seed):
            arr = np.random.default_rng(seed).integers(0, 256, (64, 64, 3), dtype=np.uint8)
            buf = io.BytesIO()
            Image.fromarray(arr).save(buf, format="PNG")
            return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()

        def ask(seed):
            msgs = [{"role": "user", "content": [{"type": "text", "text": "what is this"},
                                                 {"type": "image_url", "image_url": {"url": uri(seed)}}]}]
            req = GenRequest(messages=msgs, max_tokens=6, temperature=0.0)
            ids, pm = svc.prepare_full(req)
            assert pm is not None and ids.count(tok.token_id(M.IMAGE_PAD)) == 4 and pm.rope_delta == 2 - 4
            return svc.generate(req)

        a, b, a2 = ask(1), ask(2), ask(1)
        assert a.completion_tokens == 6 and a.error == ""
        assert a.content == a2.content                 # deterministic
        # text-only request still works next to it
        plain = svc.generate(GenRequest(messages=[{"role": "user", "content": "hello"}], max_tokens=4, temperature=0.0))
        assert plain.error == "" and plain.completion_tokens == 4
        # a prepared prompt that does not match the ids is refused at submit
        ids, pm = svc.prepare_full(GenRequest(messages=[{"role": "user", "content": [
            {"type": "image_url", "image_url": {"url": uri(3)}}]}], max_tokens=2))
        with pytest.raises(RequestError):
            engine.submit(ids[:-1], RequestOptions(max_tokens=2, media=pm))
        # remote URLs are refused with a request error
        bad = GenRequest(messages=[{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "http://x/y.png"}}]}])
        with pytest.raises(RequestError):
            svc.prepare_full(bad)
    finally:
        engine.shutdown()

    text_engine = Engine(lambda: ReferenceProgram(cfg, w, max_lanes=2, max_context=512), prefill_chunk=16)
    try:
        svc2 = GenerationService(text_engine, tok, "tiny-dense:test")
        with pytest.raises(RequestError):
            svc2.prepare_full(GenRequest(messages=[{"role": "user", "content": [
                {"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}]}]))
    finally:
        text_engine.shutdown()
