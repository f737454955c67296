"""Generate golden vectors from the reference's own CPU-capable functions.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/MOD-DiT

The reference's `MoD.mod.attn_mask` imports third-party GPU packages that are not needed by its
CPU functions; empty stub modules are registered for them before the import.  Nothing here is
needed at test time: the tests only read the `.npz` files this script writes next to itself.
"""
from __future__ import annotations

import argparse
import contextlib
import io
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _stub(name, **attrs):
    mod = types.ModuleType(name)
    for key, val in attrs.items():
        setattr(mod, key, val)
    sys.modules[name] = mod
    return mod


def import_reference(path):
    sys.path.insert(0, path)
    _stub("sageattention", sageattn=None)
    _stub("spas_sage_attn", block_sparse_sage2_attn_cuda=None, spas_sage2_attn_meansim_topk_cuda=None)
    mpl = _stub("matplotlib")
    mpl.pyplot = _stub("matplotlib.pyplot")
    import MoD.mod.attn_mask as am
    import MoD.mod.cuda_lstsq as ls
    import MoD.mod.state as st
    import MoD.mod.triton_flash_sparsity as tf
    return am, ls, st, tf


def locality_inputs(seed, H, T, Hh, Ww, D, gain=2.0, text=0, text_first=False):
    """Small seeded q,k,v with spatio-temporal locality (fp32)."""
    g = torch.Generator().manual_seed(seed)
    t, y, x = torch.meshgrid(torch.arange(T), torch.arange(Hh), torch.arange(Ww), indexing="ij")
    pos = torch.stack([t.flatten() / max(T, 1), y.flatten() / Hh, x.flatten() / Ww], 1).float()
    freqs = 2.0 ** torch.arange(8).float()
    ang = pos[:, :, None] * freqs[None, None, :] * math.pi
    pe = torch.cat([ang.sin(), ang.cos()], -1).reshape(pos.shape[0], -1)            # (Nv,48)
    W = torch.randn(H, 48, D, generator=g) / 48 ** 0.5
    nv = pos.shape[0]
    q = 0.5 * torch.randn(H, nv, D, generator=g) + gain * torch.einsum("np,hpd->hnd", pe, W)
    k = 0.5 * torch.randn(H, nv, D, generator=g) + gain * torch.einsum("np,hpd->hnd", pe, W)
    v = torch.randn(H, nv, D, generator=g)
    if text:
        tq, tk, tv = (torch.randn(H, text, D, generator=g) for _ in range(3))
        cat = (lambda a, b: torch.cat([b, a], 1)) if text_first else (lambda a, b: torch.cat([a, b], 1))
        q, k, v = cat(q, tq), cat(k, tk), cat(v, tv)
    return q[None], k[None], v[None]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MODDIT_REFERENCE", ""),
                    help="path of the reference checkout (or set MODDIT_REFERENCE)")
    args = ap.parse_args()
    if not args.reference or not os.path.isdir(os.path.join(args.reference, "MoD")):
        ap.error("--reference must point to a MOD-DiT checkout (the directory that holds MoD/)")
    am, ls, st, tf = import_reference(args.reference)
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---- 1. sparsity map + dense output from the reference's CPU path (three layouts) -------------
    out = {}
    cases = [
        ("hunyuan", 64, dict(H=2, T=2, Hh=8, Ww=16, D=64, text=64, text_first=False)),
        ("cogvideox", 64, dict(H=2, T=2, Hh=8, Ww=16, D=64, text=64, text_first=True)),
        ("wan", 64, dict(H=2, T=2, Hh=8, Ww=16, D=64, text=0)),
        ("hunyuan", 128, dict(H=1, T=3, Hh=8, Ww=16, D=128, text=128, text_first=False)),
    ]
    for ci, (model_type, bs, kw) in enumerate(cases):
        q, k, v = locality_inputs(100 + ci, **kw)
        S = q.shape[2]
        text = kw.get("text", 0)
        video = S - text
        thr = 1e-3
        if model_type == "wan":
            # the reference CPU function has no 'wan' branch; the hunyuan branch with no text is the same layout
            o, m = am._compute_block_sparse_map(q, k, v, block_size=bs, video_token_num=video,
                                                text_token_num=0, threshold=thr, model_type="hunyuan")
        else:
            o, m = am._compute_block_sparse_map(q, k, v, block_size=bs, video_token_num=video,
                                                text_token_num=text, threshold=thr, model_type=model_type)
        o2, m2 = tf._naive_attn_with_sparsity(q, k, v, thr, bs, model_type=model_type,
                                              video_token_num=video, text_token_num=text)
        out[f"map{ci}_q"], out[f"map{ci}_k"], out[f"map{ci}_v"] = q.numpy(), k.numpy(), v.numpy()
        out[f"map{ci}_out"] = o.numpy()
        out[f"map{ci}_map"] = m.float().numpy()
        out[f"map{ci}_naive_map"] = m2.float().numpy()
        out[f"map{ci}_meta"] = np.array([bs, video, text, S], dtype=np.int64)
        out[f"map{ci}_model"] = np.array(model_type)
    np.savez_compressed(os.path.join(HERE, "sparsity_map.npz"), **out)

    # ---- 2. lstsq: MTM, MTS, solve ---------------------------------------------------------------
    out = {}
    for ci, (n, bpf, H, lam) in enumerate([(12, 4, 3, 1.0), (13, 4, 2, 1.0), (32, 8, 2, 1.0), (30, 7, 2, 1e-3)]):
        g = torch.Generator().manual_seed(200 + ci)
        # maps on the reference's value grid: count / 64^2 rounded to fp16
        S_T = (torch.randint(0, 4097, (H, n, n), generator=g).float() / 4096.0).to(torch.float16)
        mtm = ls.compute_mtm_pytorch(S_T.float(), bpf, lam)
        mts = ls.compute_mts_pytorch(S_T.float(), bpf)
        state = {"warmup_steps": 4}
        with contextlib.redirect_stdout(io.StringIO()):
            feats = ls.solve_lstsq(state, S_T, step=3, blocks_per_frame=bpf, regularization=lam, use_cuda=False)
            zeros = ls.solve_lstsq(state, S_T, step=2, blocks_per_frame=bpf, regularization=lam, use_cuda=False)
        out[f"ls{ci}_S"] = S_T.float().numpy()
        out[f"ls{ci}_meta"] = np.array([n, bpf, H], dtype=np.int64)
        out[f"ls{ci}_lam"] = np.array(lam)
        out[f"ls{ci}_mtm"] = mtm.numpy()
        out[f"ls{ci}_mts"] = mts.numpy()
        out[f"ls{ci}_d"] = feats["d"].numpy()
        out[f"ls{ci}_c"] = feats["c"].numpy()
        out[f"ls{ci}_bd"] = feats["b_d"].numpy()
        out[f"ls{ci}_recon"] = ls.reconstruct_attention_map(feats, n, bpf).numpy()
        out[f"ls{ci}_zero_d_shape"] = np.array(zeros["d"].shape)
        assert float(zeros["d"].abs().sum() + zeros["c"].abs().sum() + zeros["b_d"].abs().sum()) == 0.0
    np.savez_compressed(os.path.join(HERE, "lstsq.npz"), **out)

    # ---- 3. selection + mask generation ------------------------------------------------------------
    out = {}
    sel_cases = [
        ("hunyuan", 64, 12 * 64, 2 * 64, 4, 3, 9),
        ("cogvideox", 64, 12 * 64, 2 * 64, 4, 3, 9),
        ("wan", 128, 16 * 128, 0, 4, 2, 11),
        ("hunyuan", 128, 15 * 128, 128, 5, 2, 60),   # top_k larger than the number of lines
    ]
    for ci, (model_type, bs, video, text, bpf, H, top_k) in enumerate(sel_cases):
        g = torch.Generator().manual_seed(300 + ci)
        n = video // bs
        hist = []
        for _ in range(2):
            hist.append({"c": torch.randn(H, n, generator=g), "d": torch.randn(H, 2 * n - 1, generator=g),
                         "b_d": torch.randn(H, generator=g) + 1.0})
        predict_T = 5
        lines = am.choose_topk_lines(hist, top_k=top_k, predict_T=predict_T)
        pred = torch.cat([hist[1]["c"] + (hist[1]["c"] - hist[0]["c"]) / predict_T,
                          hist[1]["d"] + (hist[1]["d"] - hist[0]["d"]) / predict_T], 1)
        state = st.create_adaptive_mask_state(model_type, H, video, text, bpf * bs, video // (bpf * bs),
                                              warmup_steps=4, top_k=top_k, predict_T=predict_T,
                                              block_size=bs)
        state["features_history"] = hist
        state["current_steps"] = 4
        with contextlib.redirect_stdout(io.StringIO()):
            info = am.predict_mask_from_warmup(state, video + text, top_k=top_k)
            modes = ["sparse", "block_diagonal", "full"][:H] + ["sparse"] * max(0, H - 3)
            mask_modes = am.generate_mask_from_lines(state, H, video + text, bpf, lines, modes, torch.device("cpu"))
        out[f"sel{ci}_model"] = np.array(model_type)
        out[f"sel{ci}_meta"] = np.array([bs, video, text, bpf, H, top_k, predict_T], dtype=np.int64)
        for t_ in range(2):
            for key in ("c", "d", "b_d"):
                out[f"sel{ci}_h{t_}_{key}"] = hist[t_][key].numpy()
        out[f"sel{ci}_pred"] = pred.numpy()
        out[f"sel{ci}_lines"] = lines.numpy()
        out[f"sel{ci}_mode"] = np.array(info["mode"])
        out[f"sel{ci}_mask"] = info["mask"].numpy()
        out[f"sel{ci}_modes2"] = np.array(modes)
        out[f"sel{ci}_mask2"] = mask_modes.numpy()
    np.savez_compressed(os.path.join(HERE, "selection.npz"), **out)

    # ---- 4. static radial masks (frames of whole, fractional and sub-block size; both model layouts) ---
    out = {}
    radial_cases = [("hunyuan", 1536, 6, 128), ("hunyuan", 1920, 5, 256), ("hunyuan", 1280, 4, 128),
                    ("wan", 1600, 8, 64), ("wan", 2560, 10, 0), ("hunyuan", 2560, 20, 128), ("wan", 3072, 12, 0),
                    ("hunyuan", 7680, 30, 256), ("wan", 6240, 13, 32)]
    for ci, (model_type, video, frames, text) in enumerate(radial_cases):
        q = torch.zeros(1, 1, video + text, 8)
        with contextlib.redirect_stdout(io.StringIO()):
            mask = am.get_radial_mask(q, video, frames, model_type=model_type)
        out[f"rad{ci}_model"] = np.array(model_type)
        out[f"rad{ci}_meta"] = np.array([video, frames, text], dtype=np.int64)
        out[f"rad{ci}_mask"] = np.packbits(mask[0].numpy())
        out[f"rad{ci}_shape"] = np.array(mask[0].shape, dtype=np.int64)
    out["count"] = np.array(len(radial_cases))
    np.savez_compressed(os.path.join(HERE, "radial.npz"), **out)

    # ---- 4b. the rotary function the Wan processor defines inside its __call__ ------------------------
    # (MoD/models/wan/attention_processor.py:78-90): the processor module needs `diffusers`, which is absent, so
    # the nested function is lifted out of the parsed file and run as it stands
    import ast
    import textwrap
    src = open(os.path.join(args.reference, "MoD", "models", "wan", "attention_processor.py")).read()
    nested = [node for node in ast.walk(ast.parse(src))
              if isinstance(node, ast.FunctionDef) and node.name == "apply_rotary_emb"]
    assert len(nested) == 1
    scope = {"torch": torch}
    exec(textwrap.dedent(ast.get_source_segment(src, nested[0])), scope)
    out = {}
    for ci, (dtype, S, Hn, Dh) in enumerate([(torch.bfloat16, 9, 2, 16), (torch.float16, 5, 3, 64),
                                             (torch.float32, 7, 1, 128)]):
        g = torch.Generator().manual_seed(500 + ci)
        x = torch.randn(2, S, Hn, Dh, generator=g).to(dtype)
        ang = torch.rand(S, Dh // 2, generator=g) * 6.28
        # tables shaped like the model's: (1, S, 1, D); even and odd entries differ on purpose
        cos = (ang.cos().repeat_interleave(2, 1) * torch.linspace(0.9, 1.1, Dh)).view(1, S, 1, Dh)
        sin = (ang.sin().repeat_interleave(2, 1) * torch.linspace(1.1, 0.9, Dh)).view(1, S, 1, Dh)
        y = scope["apply_rotary_emb"](x, cos, sin)
        assert y.dtype == dtype
        out[f"rot{ci}_dtype"] = np.array(str(dtype).replace("torch.", ""))
        out[f"rot{ci}_x"] = x.float().numpy()
        out[f"rot{ci}_cos"] = cos.view(S, Dh).numpy()
        out[f"rot{ci}_sin"] = sin.view(S, Dh).numpy()
        out[f"rot{ci}_y"] = y.float().numpy()
    out["count"] = np.array(3)
    np.savez_compressed(os.path.join(HERE, "rotary.npz"), **out)

    # ---- 5. state keys -----------------------------------------------------------------------------
    state = st.create_adaptive_mask_state("hunyuan", 24, 115200, 256, 3840, 30)
    with open(os.path.join(HERE, "state_keys.txt"), "w") as fh:
        for key in state:
            fh.write(f"{key}={state[key]!r}\n")
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
