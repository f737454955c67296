"""Drop-in `MoD` package: the `MoD.mod` modules keep the reference's names and signatures and run on the
sm_100a kernels of `moddit_b200`.

Only the hot-path modules live here.  When a checkout of the reference project is on `sys.path` behind this
directory, the rest of its `MoD` package (`MoD.models`, `MoD.inference`, `MoD.mod.utils`, `MoD.mod.logger`)
keeps resolving to the checkout: both package paths are extended over every `MoD` directory on `sys.path`,
and this directory, being first, wins for the modules it provides."""
from pkgutil import extend_path

__path__ = extend_path(__path__, __name__)
