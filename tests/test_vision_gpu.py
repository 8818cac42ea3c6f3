"""The vision tower (vlab200_vision_*): camera views -> image-token embeddings, against the CPU oracle's restatement of
the reference's SigLIP tower and connector (src/models/smolvla.cpp:394-426,1511-1563; src/models/pi0.cpp:130-155,
479-499).

Bar: rel-L2 <= 2e-2 on the embeddings of each view (bf16 operands and bf16 activations between the stages on the GPU,
float32 oracle on the same bf16-representable weights); the float32 residual stream keeps the distance flat over
depth.  The same bar as the prefix K/V."""
import numpy as np
import pytest

from tests.gpu_util import bits_to_bf16_tensor, rel_l2, require_cuda, to_dev

pytestmark = pytest.mark.gpu


def make_tower(oracle, rng, cfg, connector_bias=False):
    H, I, P, L = cfg["hidden"], cfg["inter"], cfg["patch"], cfg["n_layers"]
    n = (cfg["image"] // P) ** 2
    c4 = H * cfg["shuffle"] ** 2
    mat = lambda o, i: oracle.bf16_round((rng.standard_normal((o, i)) * i ** -0.5).astype(np.float32))
    vec = lambda k, s=0.05: (rng.standard_normal(k) * s).astype(np.float32)
    w = dict(patch_w=mat(H, 3 * P * P).reshape(H, 3, P, P), patch_b=vec(H), pos=(rng.standard_normal((n, H)) * 0.1).astype(np.float32),
             post_w=(1 + vec(H, 0.1)), post_b=vec(H), connector=mat(cfg["out_dim"], c4),
             connector_b=vec(cfg["out_dim"]) if connector_bias else None, layers=[])
    for _ in range(L):
        w["layers"].append(dict(ln1_w=1 + vec(H, 0.1), ln1_b=vec(H), ln2_w=1 + vec(H, 0.1), ln2_b=vec(H),
                                wq=mat(H, H), bq=vec(H), wk=mat(H, H), bk=vec(H), wv=mat(H, H), bv=vec(H),
                                wo=mat(H, H), bo=vec(H), fc1=mat(I, H), b1=vec(I), fc2=mat(H, I), b2=vec(H)))
    return w


def tower_to_dev(oracle, w):
    bf = lambda a: bits_to_bf16_tensor(oracle.f32_to_bf16_bits(np.ascontiguousarray(a, np.float32)))
    d = dict(patch_w=bf(w["patch_w"].reshape(w["patch_w"].shape[0], -1)), patch_b=to_dev(w["patch_b"]), pos=to_dev(w["pos"]),
             post_w=to_dev(w["post_w"]), post_b=to_dev(w["post_b"]), connector=bf(w["connector"]),
             connector_b=None if w["connector_b"] is None else to_dev(w["connector_b"]))
    for k in ("ln1_w", "ln1_b", "ln2_w", "ln2_b", "bq", "bk", "bv", "bo", "b1", "b2"):
        d[k] = [to_dev(lw[k]) for lw in w["layers"]]
    for k in ("wq", "wk", "wv", "wo", "fc1", "fc2"):
        d[k] = [bf(lw[k]) for lw in w["layers"]]
    return d


SMALL = dict(image=64, patch=16, hidden=128, n_layers=2, n_heads=2, inter=256, shuffle=2, out_dim=192, ln_eps=1e-6, out_scale=0.0)
# head_dim 72 (zero-padded to 128 inside), patch 14 (K = 588, padded to 592), connector bias and scale: pi0's tower, narrow
PI0_NARROW = dict(image=56, patch=14, hidden=288, n_layers=2, n_heads=4, inter=536, shuffle=1, out_dim=256, ln_eps=1e-6,
                  out_scale=1.0 / 16.0)
SMOLVLA = dict(image=512, patch=16, hidden=768, n_layers=12, n_heads=12, inter=3072, shuffle=4, out_dim=960, ln_eps=1e-6,
               out_scale=0.0)
PI0 = dict(image=224, patch=14, hidden=1152, n_layers=27, n_heads=16, inter=4304, shuffle=1, out_dim=2048, ln_eps=1e-6,
           out_scale=2048 ** -0.5)


@pytest.mark.parametrize("name,cfg,n_views,bias", [("small", SMALL, 2, False), ("pi0-narrow", PI0_NARROW, 3, True),
                                                   ("smolvla", SMOLVLA, 1, False), ("pi0", PI0, 2, True)])
def test_tower_matches_the_oracle(oracle, name, cfg, n_views, bias):
    torch = require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(11 + cfg["hidden"])
    w = make_tower(oracle, rng, cfg, connector_bias=bias)
    tower = vb.VisionTower(cfg, tower_to_dev(oracle, w), max_views=n_views)
    side = cfg["image"]
    g = side // cfg["patch"]
    assert tower.tokens_per_view == (g // cfg["shuffle"]) ** 2
    u8 = rng.integers(0, 256, (n_views, side, side, 3), dtype=np.uint8)
    got = tower.run(torch.from_numpy(u8).cuda()).cpu().numpy().reshape(n_views, tower.tokens_per_view, cfg["out_dim"])
    assert vb.device_status() == 0
    worst = 0.0
    for v in range(n_views):
        ref = oracle.siglip_tower(u8[v], w, cfg)
        worst = max(worst, rel_l2(got[v], ref))
    # float32 pixels in [0, 1]: the same picture gives the same embeddings bit for bit when the values are u8 / 255
    f32 = (u8.astype(np.float32) / np.float32(255.0))
    got_f = tower.run(torch.from_numpy(f32).cuda()).cpu().numpy().reshape(got.shape)
    assert np.array_equal(got, got_f)
    print(f"vision tower {name}: worst rel_l2 {worst:.3e} over {n_views} views")
    assert worst <= 2e-2, worst


def test_tower_rejects_bad_arguments(oracle):
    torch = require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(1)
    w = tower_to_dev(oracle, make_tower(oracle, rng, SMALL))
    with pytest.raises(vb.VlaB200Error):
        vb.VisionTower(dict(SMALL, image=60), w)  # not a multiple of the patch
    with pytest.raises(vb.VlaB200Error):
        vb.VisionTower(dict(SMALL, shuffle=3), w)  # the patch grid (4) is not a multiple of 3
    tower = vb.VisionTower(SMALL, w, max_views=1)
    with pytest.raises(vb.VlaB200Error):
        tower.run(torch.zeros((2, 64, 64, 3), dtype=torch.uint8, device="cuda"))  # more views than max_views
