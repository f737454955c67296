"""GPU tests of the drop-in `MoD.mod` API: validation, public map API, and the step-indexed state machine."""
import logging
import math
import os

import pytest
import torch

from oracle import moddit_oracle as orc

pytestmark = pytest.mark.gpu

LOG = logging.getLogger("moddit-test")


@pytest.fixture(scope="module")
def mod():
    import MoD.mod.attn_mask as am
    import MoD.mod.cuda_flash_sparsity as cf
    import MoD.mod.cuda_lstsq as ls
    import MoD.mod.state as st
    import MoD.mod.triton_flash_sparsity as tf
    return dict(am=am, cf=cf, ls=ls, st=st, tf=tf)


def _layout(model_type, block_size):
    if model_type == "wan":
        return block_size * 2, block_size * 2, 0
    return block_size * 3, block_size * 2, block_size


@pytest.mark.parametrize("model_type", ["hunyuan", "cogvideox", "wan"])
@pytest.mark.parametrize("block_size", [64, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_public_api_matches_probability_reference(mod, monkeypatch, model_type, block_size, dtype):
    torch.manual_seed(11)
    monkeypatch.setenv("MOD_DIT_SPARSITY_BACKEND", "triton")
    S, video, text = _layout(model_type, block_size)
    q = torch.randn(1, 2, S, 64, device="cuda", dtype=dtype)
    k, v = torch.randn_like(q), torch.randn_like(q)
    out, sp = mod["tf"].flash_attn_with_sparsity_map(
        q, k, v, 1e-3, block_size, model_type=model_type,
        video_token_num=video if model_type != "wan" else 0, text_token_num=text)
    ref_out, ref_map = orc.attn_with_sparsity_map_probs(
        q.cpu(), k.cpu(), v.cpu(), threshold=1e-3, block_size=block_size, model_type=model_type,
        video_token_num=video if model_type != "wan" else 0, text_token_num=text)
    assert out.shape == q.shape and sp.shape == ref_map.shape and sp.dtype == torch.float16
    # the reference's own bound for this comparison: 8.1 elements per block
    assert ((sp.cpu().float() - ref_map.float()).abs() * block_size ** 2).max().item() <= 8.1
    assert (out.float().cpu() - ref_out).abs().max().item() < 2e-2


def test_non_positive_threshold_produces_zero_map(mod):
    q = torch.randn(1, 1, 128, 64, device="cuda", dtype=torch.float16)
    out, sp = mod["tf"].flash_attn_with_sparsity_map(q, q, q, 0.0, 64, model_type="wan")
    assert out.shape == q.shape and torch.count_nonzero(sp).item() == 0


def test_backend_env_is_validated(mod, monkeypatch):
    q = torch.randn(1, 1, 128, 64, device="cuda", dtype=torch.float16)
    lse, scale = orc.replay_lse(q.cpu(), q.cpu())
    kw = dict(softmax_scale=scale, log_threshold=math.log(1e-3), q_video_offset=0, k_video_offset=0,
              video_blocks=2, block_size=64)
    for name in ("triton", "cuda", "auto"):
        monkeypatch.setenv("MOD_DIT_SPARSITY_BACKEND", name)
        assert mod["tf"]._compute_sparsity_map(q, q, lse.cuda(), **kw).shape == (1, 1, 2, 2)
    monkeypatch.setenv("MOD_DIT_SPARSITY_BACKEND", "invalid")
    with pytest.raises(ValueError, match="MOD_DIT_SPARSITY_BACKEND"):
        mod["tf"]._compute_sparsity_map(q, q, lse.cuda(), **kw)
    assert mod["cf"].cuda_backend_supported() and mod["cf"].extension_error() is None


@pytest.mark.parametrize("mutation,error_type,match", [
    ({"block_size": 32}, ValueError, "block_size"),
    ({"video_token_num": 65}, ValueError, "divisible"),
    ({"model_type": "unknown"}, ValueError, "Unknown model_type"),
    ({"threshold": float("nan")}, ValueError, "NaN"),
])
def test_input_validation(mod, mutation, error_type, match):
    q = torch.empty(1, 1, 128, 64, device="cuda", dtype=torch.float16)
    args = dict(query=q, key=q, value=q, threshold=1e-3, block_size=64, model_type="hunyuan",
                video_token_num=64, text_token_num=64)
    args.update(mutation)
    with pytest.raises(error_type, match=match):
        mod["tf"]._validate_inputs(**args)


def test_state_keys_match_reference(mod, golden_dir):
    state = mod["st"].create_adaptive_mask_state("hunyuan", 24, 115200, 256, 3840, 30)
    ref = [ln.split("=", 1) for ln in open(os.path.join(golden_dir, "state_keys.txt")).read().splitlines()]
    assert list(state.keys()) == [k for k, _ in ref]
    for k_, v_ in ref:
        assert repr(state[k_]) == v_
    with pytest.raises(ValueError, match="not support"):
        mod["st"].create_adaptive_mask_state("hunyuan", 24, 115200, 256, 3840, 30, sparse_type="bogus")


def _locality(seed, H, T, Hh, Ww, D, text, text_first, gain=2.0):
    from tests.golden.make_golden import locality_inputs
    q, k, v = locality_inputs(seed, H=H, T=T, Hh=Hh, Ww=Ww, D=D, gain=gain, text=text, text_first=text_first)
    return q.bfloat16(), k.bfloat16(), v.bfloat16()


@pytest.mark.parametrize("model_type,bs,text", [("hunyuan", 64, 128), ("cogvideox", 64, 128), ("wan", 128, 0),
                                                ("hunyuan", 128, 256)])
def test_state_machine_against_oracle(mod, model_type, bs, text):
    am, st = mod["am"], mod["st"]
    H, T, Hh, Ww, D = 2, 4, 16, 16, 64
    video = T * Hh * Ww                      # 1024 tokens, 256 per frame
    q0, k0, v0 = _locality(50, H, T, Hh, Ww, D, text, model_type == "cogvideox")
    S = video + text
    bpf = (Hh * Ww) // bs
    top_k, pT, warm = 6, 3, 4
    state = st.create_adaptive_mask_state(model_type, H, video, text, Hh * Ww, T, warmup_steps=warm, top_k=top_k,
                                          predict_T=pT, threshold=1e-3, block_size=bs)
    pdm = None
    valid = S
    if model_type == "hunyuan":
        valid = video + text - 37
        pdm = (torch.arange(S) < valid).unsqueeze(0).expand(S, S).contiguous().cuda()
    n = video // bs
    hist = []
    prev_map = None
    ref_mask = None
    for step in range(warm - 2, warm + 2 * pT):
        g = torch.Generator().manual_seed(1000 + step)
        q = (q0 + 0.05 * torch.randn(q0.shape, generator=g).bfloat16())
        k = (k0 + 0.05 * torch.randn(k0.shape, generator=g).bfloat16())
        out, info = am.SparseAttentionWithMap(q.cuda(), k.cuda(), v0.cuda(), state, LOG, pre_defined_mask=pdm,
                                              current_step=step)
        assert out.shape == q.shape
        refresh = step >= warm and (step - warm) % pT == pT - 1
        if step < warm or refresh:
            # dense output (all keys, as the reference's refresh pass does)
            ref = orc.masked_attention(q, k, v0, torch.ones(1, (S + bs - 1) // bs, (S + bs - 1) // bs, dtype=torch.bool), bs)
            assert (out.float().cpu() - ref).abs().max().item() < 2e-2
            cur_map = state["prev_full_maps"].cpu()
            if step >= warm:
                vm = ref_mask if model_type == "wan" else (
                    ref_mask[:, :n, :n] if model_type == "hunyuan" else ref_mask[:, text // bs:, text // bs:])
                # merged = where(mask, current, previous): where the mask was off, history must be unchanged
                assert torch.equal(cur_map[~vm], prev_map[~vm])
            prev_map = cur_map
            if step == warm - 2:
                zeros = {"c": torch.zeros(H, n), "d": torch.zeros(H, 2 * n - 1), "b_d": torch.zeros(H)}
                hist = [zeros]
            else:
                f = orc.solve_features(orc.compute_mts(cur_map, bpf), n, bpf, 1.0)
                hist.append({k_: f[k_] for k_ in ("c", "d", "b_d")})
                hist = hist[-2:]
                gpu_f = state["features_history"][-1]
                for k_ in ("c", "d", "b_d"):
                    assert torch.allclose(gpu_f[k_].cpu(), hist[-1][k_], atol=5e-4, rtol=1e-3)
                if step == warm - 1:
                    modes = orc.check_bd_values(hist[-1]["b_d"], 1.0)
                    assert state["mode"] == modes
                # bit-exact mask given identical selection inputs (the GPU's own features)
                gh = [{k_: v_.cpu() for k_, v_ in f_.items()} for f_ in state["features_history"][-2:]]
                lines = orc.choose_topk_lines(gh[0], gh[1], top_k, pT)
                ref_mask = orc.generate_mask_from_lines(
                    model_type=model_type, block_size=bs, video_token_num=video, text_token_num=text, seq_len=S,
                    blocks_per_frame=bpf, selected_lines=lines, mode=state["mode"])
                assert torch.equal(state["mask"].cpu(), ref_mask)
                # end to end (oracle features from the same map): at least 99.9 % of blocks agree
                lines2 = orc.choose_topk_lines(hist[0], hist[1], top_k, pT)
                mask2 = orc.generate_mask_from_lines(
                    model_type=model_type, block_size=bs, video_token_num=video, text_token_num=text, seq_len=S,
                    blocks_per_frame=bpf, selected_lines=lines2, mode=state["mode"])
                assert (mask2 == ref_mask).float().mean().item() >= 0.999
        else:
            kw = {}
            if pdm is not None:
                kw = dict(q_split=video, kv_len_lo=min(S, (valid + 63) // 64 * 64), kv_len_hi=valid)
            ref = orc.masked_attention(q, k, v0, ref_mask, bs, **kw)
            err = (out.float().cpu() - ref).abs()
            assert err.max().item() <= 2e-2
            assert ((out.float().cpu() - ref).norm() / ref.norm()).item() <= 1e-2
    from moddit_b200 import ops
    ops.raise_on_status(torch.device("cuda"))


def test_pooled_producer_and_mass_selector(mod):
    am, st = mod["am"], mod["st"]
    H, T, Hh, Ww, D, bs = 2, 4, 16, 16, 128, 128
    video = T * Hh * Ww
    q0, k0, v0 = _locality(60, H, T, Hh, Ww, D, 0, False)
    n, bpf = video // bs, (Hh * Ww) // bs
    for selector in ("topk_lines", "cumulative_mass"):
        state = st.create_adaptive_mask_state("wan", H, video, 0, Hh * Ww, T, warmup_steps=2, top_k=5, predict_T=4,
                                              block_size=bs)
        state["score_producer"] = "pooled"
        state["selector"] = selector
        state["mass_threshold"] = 0.9
        for step in range(0, 4):
            out, info = am.SparseAttentionWithMap(q0.cuda(), k0.cuda(), v0.cuda(), state, LOG, current_step=step)
            dark = orc.pooled_darkness_map(orc.pool_blocks(q0, bs), orc.pool_blocks(k0, bs), q_block_offset=0,
                                           k_block_offset=0, video_blocks=n, scale=D ** -0.5)[0]
            assert (state["prev_full_maps"].cpu().float() - dark.float()).abs().max().item() <= 2e-3
            if step == 0:
                ref = orc.masked_attention(q0, k0, v0, torch.ones(1, n, n, dtype=torch.bool), bs)
            else:
                gpu_dark = state["prev_full_maps"].cpu()
                if selector == "cumulative_mass":
                    ref_mask = orc.select_mass(gpu_dark, 0.9)
                else:
                    gh = [{k_: v_.cpu() for k_, v_ in f_.items()} for f_ in state["features_history"][-2:]]
                    lines = orc.choose_topk_lines(gh[0], gh[1], 5, 4)
                    modes = orc.check_bd_values(gh[1]["b_d"], 1.0)
                    ref_mask = orc.generate_mask_from_lines(
                        model_type="wan", block_size=bs, video_token_num=video, text_token_num=0, seq_len=video,
                        blocks_per_frame=bpf, selected_lines=lines, mode=modes)
                assert torch.equal(state["mask"].cpu(), ref_mask)
                ref = orc.masked_attention(q0, k0, v0, ref_mask, bs)
            assert (out.float().cpu() - ref).abs().max().item() <= 2e-2


def test_use_dense_and_unsupported_types(mod):
    am, st = mod["am"], mod["st"]
    q = torch.randn(1, 2, 512, 64, device="cuda", dtype=torch.bfloat16)
    state = st.create_adaptive_mask_state("wan", 2, 512, 0, 128, 4, block_size=64)
    out, info = am.SparseAttentionWithMap(q, q, q, state, LOG, use_dense=True, use_cuda=True)
    ref = orc.masked_attention(q.cpu(), q.cpu(), q.cpu(), torch.ones(1, 8, 8, dtype=torch.bool), 64)
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2 and info["mask"] is None
    state["sparse_type"] = "full"              # dense on every step
    full, info = am.SparseAttentionWithMap(q, q, q, state, LOG, current_step=20)
    assert torch.equal(full, out) and info["mask"] is None
    state["sparse_type"] = "svg"
    with pytest.raises(NotImplementedError):
        am.SparseAttentionWithMap(q, q, q, state, LOG, current_step=0)
    state["sparse_type"] = "radial"            # the reference builds this mask for block_size 128 only
    with pytest.raises(ValueError, match="block_size 128"):
        am.SparseAttentionWithMap(q, q, q, state, LOG, current_step=0)


@pytest.mark.parametrize("model_type,video,frames,text", [("hunyuan", 2560, 20, 128), ("hunyuan", 1280, 4, 128),
                                                          ("wan", 2560, 10, 0), ("wan", 1600, 8, 64)])
def test_radial_mask_kernel_against_oracle_and_reference(mod, golden_dir, model_type, video, frames, text):
    """`get_radial_mask` (one closed-form kernel) against the oracle and the reference's stored masks."""
    import numpy as np
    from MoD.mod.get_radial_mask import get_radial_mask
    S = video + text
    q = torch.empty(1, 3, S, 8, device="cuda", dtype=torch.bfloat16)
    mask = get_radial_mask(q, video, frames, model_type=model_type)
    assert mask.shape == (3, S // 128, S // 128) and mask.dtype == torch.bool
    want = orc.radial_mask(model_type, video, frames, S)
    assert (mask[0].cpu().numpy() == want).all() and torch.equal(mask[0], mask[2])
    g = np.load(os.path.join(golden_dir, "radial.npz"))
    hits = 0
    for ci in range(int(g["count"])):
        if str(g[f"rad{ci}_model"]) == model_type and tuple(int(x) for x in g[f"rad{ci}_meta"]) == (video, frames, text):
            shape = tuple(int(x) for x in g[f"rad{ci}_shape"])
            ref = np.unpackbits(g[f"rad{ci}_mask"])[:shape[0] * shape[1]].reshape(shape).astype(bool)
            assert (mask[0].cpu().numpy() == ref).all()
            hits += 1
    assert hits == 1
    with pytest.raises(ValueError, match="Unknown model type"):
        get_radial_mask(q, video, frames, model_type="cogvideox")


def test_radial_mask_all_stored_reference_cases(mod, golden_dir):
    import numpy as np
    from moddit_b200 import ops
    g = np.load(os.path.join(golden_dir, "radial.npz"))
    for ci in range(int(g["count"])):
        video, frames, text = (int(x) for x in g[f"rad{ci}_meta"])
        shape = tuple(int(x) for x in g[f"rad{ci}_shape"])
        ref = np.unpackbits(g[f"rad{ci}_mask"])[:shape[0] * shape[1]].reshape(shape).astype(bool)
        got = ops.radial_mask(str(g[f"rad{ci}_model"]), video, frames, video + text, torch.device("cuda"))
        assert (got.cpu().numpy() == ref).all(), ci
    # other block sizes and decay factors exist in the reference function's signature: against the oracle
    for bs, decay in ((64, 0.2), (128, 0.5), (128, 1.0)):
        got = ops.radial_mask("hunyuan", 3840, 12, 3840 + 256, torch.device("cuda"), block_size=bs, decay_factor=decay)
        assert (got.cpu().numpy() == orc.radial_mask("hunyuan", 3840, 12, 3840 + 256, bs, decay)).all(), (bs, decay)


def test_radial_state_machine(mod):
    """sparse_type='radial': dense output over all keys while warming up, then the sparse forward under the
    static mask (text padding rules of the hunyuan layout included)."""
    am, st = mod["am"], mod["st"]
    H, T, Hh, Ww, D, text = 2, 10, 16, 16, 64, 128
    video = T * Hh * Ww                                   # 2560 tokens, 256 per frame
    q, k, v = _locality(7, H, T, Hh, Ww, D, text, False)
    S = video + text
    state = st.create_adaptive_mask_state("hunyuan", H, video, text, Hh * Ww, T, warmup_steps=2, block_size=128,
                                          sparse_type="radial")
    valid = S - 29
    pdm = (torch.arange(S) < valid).unsqueeze(0).expand(S, S).contiguous().cuda()
    want_mask = torch.from_numpy(orc.radial_mask("hunyuan", video, T, S))
    dense = orc.masked_attention(q, k, v, torch.ones(1, S // 128, S // 128, dtype=torch.bool), 128)
    for step in range(4):
        out, info = am.SparseAttentionWithMap(q.cuda(), k.cuda(), v.cuda(), state, LOG, pre_defined_mask=pdm,
                                              current_step=step)
        if step < 2:
            assert info == {"mode": "warmup", "mask": None}
            assert (out.float().cpu() - dense).abs().max().item() <= 2e-2
        else:
            assert torch.equal(info["mask"][0].cpu(), want_mask) and info["mask"].shape[0] == H
            ref = orc.masked_attention(q, k, v, want_mask[None], 128, q_split=video,
                                       kv_len_lo=min(S, (valid + 63) // 64 * 64), kv_len_hi=valid)
            assert (out.float().cpu() - ref).abs().max().item() <= 2e-2
    assert not bool(want_mask.all())


def test_reference_named_map_functions_and_helpers(mod, capsys):
    """`_compute_block_sparse_map` / `compute_block_sparse_map` / `compute_block_sparse_map_triton` are three
    names of one computation in the reference (:152-263); the memory helpers keep their names too."""
    am = mod["am"]
    torch.manual_seed(5)
    q = torch.randn(1, 2, 384, 64, device="cuda", dtype=torch.bfloat16)
    k, v = torch.randn_like(q), torch.randn_like(q)
    state = dict(block_size=64, video_token_num=256, text_token_num=128, threshold=1e-3, model_type="hunyuan")
    a_out, a_map = am.compute_block_sparse_map(q, k, v, state)
    b_out, b_map = am._compute_block_sparse_map(q, k, v, q_chunk_blocks=2, **state)
    c_out, c_map = am.compute_block_sparse_map_triton(q, k, v, state)
    assert torch.equal(a_out, b_out) and torch.equal(a_map, b_map) and torch.equal(a_out, c_out)
    assert a_map.shape == (1, 2, 4, 4) and a_map.dtype == torch.float16
    am.reset_peak_gpu_stats()
    am.reset_peak_gpu_stats(q.device)
    am.print_peak_gpu_stats("after map:", q.device)
    assert "peak_alloc=" in capsys.readouterr().out
    assert am.get_cuda_arch_versions()[0] == "sm100"


def test_module_self_test_runs(mod, capsys):
    """`test_correctness` of the map module (the reference runs it from `__main__`, :372-400, 446-452)."""
    tf = mod["tf"]
    for model in ("hunyuan", "cogvideox"):
        for bs in (64, 128):
            tf.test_correctness(block_size=bs, D=128, model_type=model)
    assert capsys.readouterr().out.count("Sparsity max error") == 4
    tf.benchmark(H=2, S=1024, warmup=1, rep=2)


@pytest.mark.parametrize("model_type,text,producer", [("wan", 0, "replay"), ("cogvideox", 128, "replay"),
                                                      ("wan", 0, "pooled")])
def test_two_guidance_branches_in_one_call_equal_two_calls(mod, model_type, text, producer):
    """`SparseAttentionWithMapCFG` (branches folded into heads, one launch per kernel) against the way the
    reference's Wan / CogVideoX processors do it: one call and one state per branch.  Outputs and masks bit-equal
    on every step: dense warm-up, collecting steps, sparse steps and a refresh."""
    am, st = mod["am"], mod["st"]
    H, T, Hh, Ww, D, bs = 2, 4, 16, 16, 64, 64
    video = T * Hh * Ww
    S = video + text
    branches = [_locality(70 + b, H, T, Hh, Ww, D, text, model_type == "cogvideox") for b in range(2)]
    q, k, v = (torch.cat([br[i] for br in branches], dim=0).cuda() for i in range(3))       # (2, H, S, D)
    warm, pT = 3, 3

    def new_state():
        s_ = st.create_adaptive_mask_state(model_type, H, video, text, Hh * Ww, T, warmup_steps=warm, top_k=6,
                                           predict_T=pT, threshold=1e-3, block_size=bs)
        s_["score_producer"] = producer
        return s_
    single, both = [new_state(), new_state()], [new_state(), new_state()]
    for step in range(0, warm + pT + 1):
        g = torch.Generator(device="cuda").manual_seed(500 + step)
        qs = q + 0.05 * torch.randn(q.shape, device="cuda", generator=g).bfloat16()
        outs = [am.SparseAttentionWithMap(qs[b:b + 1], k[b:b + 1], v[b:b + 1], single[b], LOG, current_step=step)[0]
                for b in range(2)]
        out2, _ = am.SparseAttentionWithMapCFG(qs, k, v, both, LOG, current_step=step)
        assert out2.shape == qs.shape
        for b in range(2):
            assert torch.equal(out2[b:b + 1], outs[b]), (step, b)
            ma, mb = single[b].get("mask"), both[b].get("mask")
            assert (ma is None) == (mb is None)
            if ma is not None:
                assert torch.equal(ma, mb), (step, b)
            if single[b].get("features_history"):
                for fa, fb in zip(single[b]["features_history"], both[b]["features_history"]):
                    assert all(torch.equal(fa[k_], fb[k_]) for k_ in fa)
    assert both[0]["mask"] is not None and not bool(both[0]["mask"].all())
    with pytest.raises(ValueError, match="differ in 'top_k'"):
        other = new_state()
        other["top_k"] = 7
        am.SparseAttentionWithMapCFG(q, k, v, [new_state(), other], LOG, current_step=0)
    from moddit_b200 import ops
    ops.check_health(torch.device("cuda"))
