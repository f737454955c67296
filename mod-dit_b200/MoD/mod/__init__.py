"""Hot-path modules of `MoD.mod` on the sm_100a kernels; every other `MoD.mod.*` module (`utils`, `logger`)
resolves to the reference checkout found on `sys.path`, if there is one."""
from pkgutil import extend_path

__path__ = extend_path(__path__, __name__)
