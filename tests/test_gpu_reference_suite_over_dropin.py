"""The reference's OWN test files, run unmodified on the GPU with this repository's `muillm_ext` replacement registered
under that name: `MuiLinear`, `MuiMultiLinear`, `MuiGateUpDownMLP`, `MuiRMSNorm`, `MuiGateUpDownMLPMoe`, the KV caches,
the rotary embedding, the L2 norm, temperature tuning and the embedding module, each compared by the reference's tests
with the Hugging Face / torch module it replaces. That is how the reference proves itself; here it proves the drop-in.

Every failure of the child run is classified: a test whose failure text matches NOT_THE_DROPIN (CPU-tensor variants,
which this library refuses by design, and the reference's own incompatibilities with the installed transformers
release) is reported and left aside; any other failure fails this test, and at least 30 of the reference's tests have
to run to completion.

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
# Failures that say nothing about the drop-in: (text in the failure, why)
NOT_THE_DROPIN = [
    ("must be a CUDA tensor", "CPU tensors: this library has no CPU path and refuses them, the reference falls back to torch"),
    ("KeyError: 'default'", "the reference's rotary module indexes transformers' ROPE_INIT_FUNCTIONS['default'], gone "
                            "from newer transformers releases"),
    ("KeyError: 'factor'", "the reference's Llama-4 rotary set-up reaches transformers' llama3 RoPE initialiser with the "
                           "older `rope_scaling` layout (raised inside transformers/modeling_rope_utils.py)"),
    ("has no attribute 'key_cache'", "the reference's caches read `key_cache` / `value_cache` of transformers' Cache "
                                     "classes, gone from newer transformers releases"),
    ("tensor_parallelism 1 is bigger than number of available devices", "no GPU visible"),
]

FILES = ["test_linear.py", "test_multilinear.py", "test_gateupdownmlp.py", "test_rmsnorm.py", "test_l2norm.py",
         "test_gateupdownmlpmoe.py", "test_temperaturetuning.py", "test_embedding.py", "test_rotaryembedding.py",
         "test_static_kvcache.py", "test_dynamic_kvcache.py", "test_hybridchunked_kvcache.py"]


@pytest.mark.skipif(not (REF and os.path.isdir(os.path.join(REF, "muillm")) and os.path.isdir(os.path.join(REF, "tests"))),
                    reason="no reference checkout at $MUILLM_REFERENCE")
def test_reference_test_files_pass_over_the_dropin(tmp_path):
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
    xml = os.path.join(tmp_path, "reference_suite.xml")
    r = subprocess.run([sys.executable, "-m", "pytest", "-p", "dropin_plugin", "-p", "no:cacheprovider", "-q", "-rf",
                        f"--junitxml={xml}", *files], cwd=ref, env=env, capture_output=True, text=True, timeout=1500)
    tail = "\n".join(r.stdout.strip().splitlines()[-60:])
    print(tail)
    assert os.path.isfile(xml), f"the child pytest wrote no report:\n{tail}\n{r.stderr[-2000:]}"

    import xml.etree.ElementTree as ET

    passed, environment, real = 0, {}, []
    for case in ET.parse(xml).getroot().iter("testcase"):
        bad = [e for e in case if e.tag in ("failure", "error")]
        if not bad:
            passed += 0 if any(e.tag == "skipped" for e in case) else 1
            continue
        text = " ".join((e.get("message") or "") + " " + (e.text or "") for e in bad)
        why = next((label for needle, label in NOT_THE_DROPIN if needle in text), None)
        name = f"{case.get('classname')}::{case.get('name')}"
        if why is None:
            real.append(f"{name}: {text[:300]}")
        else:
            environment.setdefault(why, []).append(name)
    for why, names in environment.items():
        print(f"not run to completion ({why}): {len(names)} tests")
    print(f"passed over the drop-in: {passed}")
    assert not real, "the reference's tests fail over the drop-in:\n" + "\n".join(real)
    assert passed >= 30, f"only {passed} of the reference's tests ran to completion:\n{tail}"
