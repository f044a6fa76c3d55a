"""pytest plugin (`-p dropin_plugin`): registers this repository's muillm_ext replacement under the module name the
reference's Python package imports, before any test module of the reference is collected."""
import sys

from muillm_b200 import muillm_ext as _shim

sys.modules.setdefault("muillm_ext", _shim)
