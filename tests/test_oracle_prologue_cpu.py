"""CPU checks of the oracle's attention-prologue restatement against independent formulations (the third-party
functions it restates are not available to pin it against: see the docstrings in oracle/moddit_oracle.py)."""
import torch

from oracle import moddit_oracle as orc


def _inputs(dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(21)
    B, S, H, D = 2, 37, 3, 64
    q, k, v = [torch.randn(B, S, H * D, generator=g).to(dtype) for _ in range(3)]
    ang = torch.rand(S, D // 2, generator=g) * 6.28
    return (B, S, H, D), (q, k, v), ang


def test_rotation_equals_complex_multiplication():
    (B, S, H, D), (q, k, v), ang = _inputs()
    cos, sin = ang.cos().repeat_interleave(2, 1), ang.sin().repeat_interleave(2, 1)
    a = orc.qkv_prologue(q, k, v, num_heads=H, rope_cos=cos, rope_sin=sin)
    b = orc.qkv_prologue(q, k, v, num_heads=H, rope_cos=cos, rope_sin=sin, rope_form="even_cos_odd_sin")
    for x, y in zip(a, b):       # with tables repeated over the pair the two forms are one function
        assert torch.equal(x, y)
    z = torch.view_as_complex(q.double().unflatten(2, (H, D // 2, 2)).transpose(1, 2).contiguous())
    want = torch.view_as_real(z * torch.polar(torch.ones_like(ang.double()), ang.double())[None, None]).flatten(3)
    assert (a[0].double() - want).abs().max() <= 2.0 ** -8 * want.abs().max()
    assert torch.equal(a[2], v.unflatten(2, (H, D)).transpose(1, 2))


def test_rms_norm_matches_torch_rms_norm_to_one_rounding():
    (B, S, H, D), (q, k, v), _ = _inputs()
    w = (1 + 0.1 * torch.randn(D)).bfloat16()
    got = orc.qkv_prologue(q, k, v, num_heads=H, norm="rms_head", q_weight=w, k_weight=w, eps=1e-6)[0]
    x = q.unflatten(2, (H, D)).transpose(1, 2).float()
    want = torch.nn.functional.rms_norm(x, (D,), w.float(), 1e-6)
    assert (got.float() - want).abs().max() <= 2.0 ** -7 * want.abs().max()
    wa = (1 + 0.1 * torch.randn(H * D)).bfloat16()
    got = orc.qkv_prologue(q, k, v, num_heads=H, norm="rms_all_heads", q_weight=wa, k_weight=wa, eps=1e-6)[1]
    want = torch.nn.functional.rms_norm(k.float(), (H * D,), wa.float(), 1e-6).unflatten(2, (H, D)).transpose(1, 2)
    assert (got.float() - want).abs().max() <= 2.0 ** -7 * want.abs().max()


def test_rotary_range_leaves_other_tokens_alone():
    (B, S, H, D), (q, k, v), ang = _inputs()
    cos, sin = ang.cos().repeat_interleave(2, 1), ang.sin().repeat_interleave(2, 1)
    plain = orc.qkv_prologue(q, k, v, num_heads=H)
    part = orc.qkv_prologue(q, k, v, num_heads=H, rope_cos=cos[:20], rope_sin=sin[:20], rope_range=(10, 30))
    full = orc.qkv_prologue(q, k, v, num_heads=H, rope_cos=cos, rope_sin=sin)
    assert torch.equal(part[0][:, :, :10], plain[0][:, :, :10]) and torch.equal(part[0][:, :, 30:], plain[0][:, :, 30:])
    shifted = orc.qkv_prologue(q[:, 10:30], k[:, 10:30], v[:, 10:30], num_heads=H, rope_cos=cos[:20], rope_sin=sin[:20])
    assert torch.equal(part[1][:, :, 10:30], shifted[1])


def test_wan_rotary_function_matches_the_reference(golden_dir):
    """`_rope_even_cos_odd_sin` against outputs of the function the reference's Wan processor defines
    (stored by tests/golden/make_golden.py, which runs that function as it stands): bit-exact, and through
    `qkv_prologue` as well."""
    import os

    import numpy as np
    g = np.load(os.path.join(golden_dir, "rotary.npz"), allow_pickle=False)
    for ci in range(int(g["count"])):
        dtype = getattr(torch, str(g[f"rot{ci}_dtype"]))
        x = torch.from_numpy(g[f"rot{ci}_x"]).to(dtype)                 # (B, S, H, D)
        cos, sin = torch.from_numpy(g[f"rot{ci}_cos"]), torch.from_numpy(g[f"rot{ci}_sin"])
        want = torch.from_numpy(g[f"rot{ci}_y"]).to(dtype)
        assert torch.equal(orc._rope_even_cos_odd_sin(x, cos, sin), want)
        if dtype == torch.float32:
            continue
        B, S, Hn, Dh = x.shape
        flat = x.reshape(B, S, Hn * Dh)
        got = orc.qkv_prologue(flat, flat, flat, num_heads=Hn, rope_cos=cos, rope_sin=sin,
                               rope_form="even_cos_odd_sin")[0]
        assert torch.equal(got, want.transpose(1, 2))
