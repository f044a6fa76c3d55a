"""The reference's OWN test files, run unmodified on the GPU with this repository's `muillm_ext` replacement registered
under that name: `MuiLinear`, `MuiMultiLinear`, `MuiGateUpDownMLP`, `MuiRMSNorm`, `MuiGateUpDownMLPMoe`, the KV caches,
the rotary embedding, the L2 norm, temperature tuning and the embedding module, each compared by the reference's tests
with the Hugging Face / torch module it replaces. That is how the reference proves itself; here it proves the drop-in.

Needs a checkout of the reference (its `muillm/` package and `tests/`) at $MUILLM_REFERENCE; skipped where there is
none. The tests run in a child pytest with `-p dropin_plugin` (tests/dropin_plugin.py), which puts the replacement
into `sys.modules["muillm_ext"]` before the reference's modules import it."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.environ.get("MUILLM_REFERENCE", "")

# single-GPU test files of the reference (its multi-GPU files spawn one process per visible GPU on a fixed port)
FILES = ["test_linear.py", "test_multilinear.py", "test_gateupdownmlp.py", "test_rmsnorm.py", "test_l2norm.py",
         "test_gateupdownmlpmoe.py", "test_temperaturetuning.py", "test_embedding.py", "test_rotaryembedding.py",
         "test_static_kvcache.py", "test_dynamic_kvcache.py", "test_hybridchunked_kvcache.py"]


@pytest.mark.skipif(not (REF and os.path.isdir(os.path.join(REF, "muillm")) and os.path.isdir(os.path.join(REF, "tests"))),
                    reason="no reference checkout at $MUILLM_REFERENCE")
def test_reference_test_files_pass_over_the_dropin():
    ref = os.path.abspath(REF)
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, HERE, ref, env.get("PYTHONPATH", "")])
    import transformers.cache_utils as hf_cache

    names = list(FILES)
    if not hasattr(hf_cache, "HybridChunkedCache"):
        # the installed transformers no longer has the class this file compares with (see tests/dropin_plugin.py)
        names.remove("test_hybridchunked_kvcache.py")
    files = [os.path.join("tests", f) for f in names if os.path.isfile(os.path.join(ref, "tests", f))]
    assert files, "the checkout has none of the expected test files"
    r = subprocess.run([sys.executable, "-m", "pytest", "-p", "dropin_plugin", "-p", "no:cacheprovider", "-q", "-rf",
                        *files], cwd=ref, env=env, capture_output=True, text=True, timeout=1500)
    tail = "\n".join(r.stdout.strip().splitlines()[-40:])
    print(tail)
    assert r.returncode == 0, f"the reference's tests over the drop-in:\n{tail}\n{r.stderr[-2000:]}"
