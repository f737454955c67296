"""The drop-in route "put mod-dit_b200/ first on sys.path": this package's MoD.mod modules shadow the
checkout's, and everything this package does not provide still resolves to the checkout."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "mod-dit_b200")


def _run(code, extra_path):
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([PKG, extra_path]))
    return subprocess.run([sys.executable, "-c", textwrap.dedent(code)], env=env, capture_output=True, text=True)


def test_checkout_modules_resolve_behind_the_dropin(tmp_path):
    """A stand-in checkout laid out like the reference (MoD/__init__.py, MoD/mod without __init__.py,
    MoD/models/<model>/attention_processor.py importing from MoD.mod.utils and MoD.mod.attn_mask)."""
    co = tmp_path / "checkout"
    (co / "MoD" / "mod").mkdir(parents=True)
    (co / "MoD" / "models" / "hunyuan").mkdir(parents=True)
    (co / "MoD" / "__init__.py").write_text("")
    (co / "MoD" / "mod" / "utils.py").write_text("def reset_peak_gpu_stats():\n    return 'checkout utils'\n")
    (co / "MoD" / "mod" / "state.py").write_text("raise RuntimeError('the checkout state module must be shadowed')\n")
    (co / "MoD" / "models" / "__init__.py").write_text("")
    (co / "MoD" / "models" / "hunyuan" / "__init__.py").write_text("")
    (co / "MoD" / "models" / "hunyuan" / "attention_processor.py").write_text(textwrap.dedent("""
        from MoD.mod.utils import reset_peak_gpu_stats
        from MoD.mod.attn_mask import SparseAttentionWithMap
        from MoD.mod.state import create_adaptive_mask_state
        MARK = reset_peak_gpu_stats()
    """))
    res = _run("""
        import MoD.models.hunyuan.attention_processor as ap
        import MoD.mod.attn_mask as am, MoD.mod.state as st, MoD.mod.utils as ut
        print(ap.MARK)
        print(am.__file__)
        print(st.__file__)
        print(ut.__file__)
    """, str(co))
    assert res.returncode == 0, res.stderr
    mark, am_file, st_file, ut_file = res.stdout.strip().splitlines()[-4:]
    assert mark == "checkout utils"
    assert am_file.startswith(PKG) and st_file.startswith(PKG)
    assert ut_file.startswith(str(co))


def test_reference_checkout_utils_and_logger_resolve():
    """With the real checkout present (the build container only): its utils and logger modules import."""
    import pytest
    ref = os.environ.get("MODDIT_REFERENCE_CHECKOUT", os.path.join(os.sep, "root", "reference"))
    if not os.path.isdir(os.path.join(ref, "MoD", "mod")):
        pytest.skip("no reference checkout on this machine")
    res = _run("""
        import MoD.mod.utils as ut, MoD.mod.logger as lg, MoD.mod.state as st
        print(ut.__file__); print(lg.__file__); print(st.__file__)
    """, ref)
    assert res.returncode == 0, res.stderr
    ut_file, lg_file, st_file = res.stdout.strip().splitlines()[-3:]
    assert ut_file.startswith(ref) and lg_file.startswith(ref) and st_file.startswith(PKG)
