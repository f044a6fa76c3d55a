"""pytest plugin (`-p dropin_plugin`): registers this repository's muillm_ext replacement under the module name the
reference's Python package imports, before any test module of the reference is collected.

The reference's `muillm/modules/kvcache/cache_utils.py` imports `HybridChunkedCache` from `transformers.cache_utils` at
module level; newer transformers releases no longer have that class. Where it is missing, a placeholder of that name is
put there so that the modules which merely import it (static / dynamic caches, rotary embedding, temperature tuning)
still load; constructing the placeholder raises, so a test that needs the real class fails visibly."""
import sys

from muillm_b200 import muillm_ext as _shim

sys.modules.setdefault("muillm_ext", _shim)

try:
    import transformers.cache_utils as _cu

    if not hasattr(_cu, "HybridChunkedCache"):
        class HybridChunkedCache(_cu.Cache):  # noqa: D401 - placeholder, see the module docstring
            def __init__(self, *args, **kwargs):
                raise NotImplementedError("this transformers release has no HybridChunkedCache")

        _cu.HybridChunkedCache = HybridChunkedCache
        HAVE_HF_HYBRID_CHUNKED_CACHE = False
    else:
        HAVE_HF_HYBRID_CHUNKED_CACHE = True
except ImportError:  # no transformers: the reference's tests cannot run at all
    HAVE_HF_HYBRID_CHUNKED_CACHE = False
