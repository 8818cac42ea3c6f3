"""The oracle's vision-tower pieces (CPU): image preprocessing and the pixel-shuffle order against the reference's own
header compiled into oracle/_ref/libpreprocess_ref.so (when it was built) and against the known answers of the
reference's unit test (tests/test_vision_common.cpp:27-69, read as text); LayerNorm and the patch embedding against
direct float64 / loop forms."""
import ctypes as C
import os

import numpy as np
import pytest

REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libpreprocess_ref.so")


def test_pixel_shuffle_known_answers_of_the_reference_test(oracle):
    # embed 2, grid 4, s 2; src[p][e] = 1000 p + e
    embed, grid, s = 2, 4, 2
    src = (1000.0 * np.arange(grid * grid)[:, None] + np.arange(embed)[None, :]).astype(np.float32)
    dst = oracle.pixel_shuffle_hf(src, grid, s)
    assert dst.shape == (4, 8)
    assert dst[0].tolist() == [0, 1, 1000, 1001, 4000, 4001, 5000, 5001]
    assert dst[1, 0] == 2000.0
    g2 = grid // s
    for h2 in range(g2):
        for w2 in range(g2):
            for hs in range(s):
                for ws in range(s):
                    for e in range(embed):
                        p = (h2 * s + hs) * grid + (w2 * s + ws)
                        assert dst[h2 * g2 + w2, (hs * s + ws) * embed + e] == 1000.0 * p + e


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="oracle/_ref/libpreprocess_ref.so was not built")
def test_preprocess_and_pixel_shuffle_match_the_reference_header(oracle):
    L = C.CDLL(REF_LIB)
    L.ref_preprocess_image_chw.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    L.ref_pixel_shuffle_hf.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
    rng = np.random.default_rng(5)
    for side in (16, 64, 224):
        u8 = rng.integers(0, 256, (side, side, 3), dtype=np.uint8)
        f32 = rng.random((side, side, 3), dtype=np.float32)
        for img in (u8, f32):
            out = np.empty((3, side, side), np.float32)
            assert L.ref_preprocess_image_chw(img.ctypes.data, int(img.dtype == np.float32), side, out.ctypes.data) == 1
            assert np.array_equal(out, oracle.preprocess_image_chw(img))
    for embed, grid, s in ((2, 4, 2), (8, 8, 4), (24, 32, 4), (5, 6, 3), (7, 4, 1)):
        src = rng.standard_normal((grid * grid, embed)).astype(np.float32)
        dst = np.empty(((grid // s) ** 2, embed * s * s), np.float32)
        L.ref_pixel_shuffle_hf(src.ctypes.data, dst.ctypes.data, embed, grid, s)
        assert np.array_equal(dst, oracle.pixel_shuffle_hf(src, grid, s))


def test_layer_norm_and_patch_embedding(oracle):
    rng = np.random.default_rng(6)
    x = (rng.standard_normal((9, 96)) * 3 + 1).astype(np.float32)
    w, b = rng.standard_normal(96).astype(np.float32), rng.standard_normal(96).astype(np.float32)
    x64 = x.astype(np.float64)
    want = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-6) * w + b
    assert np.allclose(oracle.layer_norm(x, w, b, 1e-6), want, rtol=0, atol=2e-5)
    # the stride-P convolution as a linear map over flattened patches, against the direct loop
    side, P, H = 8, 4, 5
    img = rng.random((side, side, 3), dtype=np.float32)
    pw = rng.standard_normal((H, 3, P, P)).astype(np.float32)
    cfg = dict(image=side, patch=P, hidden=H, n_heads=1, shuffle=1, ln_eps=1e-6)
    chw = oracle.preprocess_image_chw(img)
    g = side // P
    direct = np.zeros((g * g, H), np.float64)
    for gy in range(g):
        for gx in range(g):
            for o in range(H):
                direct[gy * g + gx, o] = np.sum(pw[o].astype(np.float64) * chw[:, gy * P:(gy + 1) * P, gx * P:(gx + 1) * P])
    # a tower with no layers, identity post-LayerNorm weights and an identity connector exposes the embedding
    w0 = dict(patch_w=pw, patch_b=np.zeros(H, np.float32), pos=np.zeros((g * g, H), np.float32), layers=[],
              post_w=np.ones(H, np.float32), post_b=np.zeros(H, np.float32), connector=np.eye(H, dtype=np.float32))
    got = oracle.siglip_tower(img, w0, cfg)
    assert np.allclose(got, oracle.layer_norm(direct.astype(np.float32), w0["post_w"], w0["post_b"], 1e-6), atol=1e-4)
