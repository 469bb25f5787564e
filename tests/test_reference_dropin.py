"""The drop-in against the reference's own runtime: with the overlay packages of integration/ on the path and the three
registry edits applied (integration/enable_b200.py), the reference's `import_decode_schedule(model, "B200", batch)`
(qimeng_megakernel/models/LLM/registry.py:238-262) resolves to the B200 packages and yields what `_decode_mk`
(decode.py:600-642) reads: get_mk, call_mk, Globals, the config class and STATIC_MEGAKERNEL, which selects the branch
that builds no instruction queues and never zeroes a barrier tensor.  Needs an importable reference checkout (found
through QMK_REFERENCE_ROOT, else a directory `reference` beside this repository); skipped elsewhere.  No GPU and no kernel launch."""
import importlib
import inspect
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def reference_registry():
    ref = os.environ.get("QMK_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
    if not os.path.isdir(os.path.join(ref, "qimeng_megakernel")):
        pytest.skip("no reference checkout on this machine")
    for p in (ref, os.path.join(ROOT, "integration")):
        if p not in sys.path:
            sys.path.insert(0, p)
    try:
        registry = importlib.import_module("qimeng_megakernel.models.LLM.registry")
    except Exception as e:      # the reference's own imports failed (missing dependency)
        pytest.skip(f"reference not importable here: {e}")
    import enable_b200
    enable_b200.enable()
    enable_b200.enable()        # idempotent
    return registry


@pytest.mark.parametrize("model,batch,package", [
    ("meta-llama/Llama-3.2-1B-Instruct", 1, "llama.llama3_2__1b.B200.single_batch.decode_schedule"),
    ("llama-3.2-1b", 8, "llama.llama3_2__1b.B200.multi_batch.decode_schedule"),
    ("llama-3.2-1b", 64, "llama.llama3_2__1b.B200.multi_batch.decode_schedule"),
    ("Qwen/Qwen3-0.6B", 1, "qwen.qwen3__0_6b.B200.single_batch.decode_schedule"),
    ("qwen3-0.6b", 16, "qwen.qwen3__0_6b.B200.multi_batch.decode_schedule"),
])
def test_reference_registry_resolves_the_b200_packages(reference_registry, model, batch, package):
    import qimeng_megakernel_b200 as ours
    sched = reference_registry.import_decode_schedule(model, "B200", batch)
    assert sched.package_name == "qimeng_megakernel.models.LLM." + package
    assert sched.get_mk is ours.mk_kernel.get_mk and sched.call_mk is ours.mk_kernel.call_mk
    assert sched.globs_cls is ours.Globals and sched.config is ours.LlamaConfig
    assert getattr(sched.package, "STATIC_MEGAKERNEL") is True
    assert sched.scheduler is None and sched.python_vm is None      # nothing to build or tensorise


def test_reference_runtime_keys_on_the_static_flag(reference_registry):
    decode = importlib.import_module("qimeng_megakernel.models.LLM.decode")
    src = inspect.getsource(decode._decode_mk)
    assert 'getattr(schedule.package, "STATIC_MEGAKERNEL", False)' in src.replace("\n", "").replace("  ", "") or \
        "STATIC_MEGAKERNEL" in src
    assert "if not static_megakernel" in src        # queue building and tensorising sit behind the flag
    # the other hardware keeps resolving as before, and the caps hold
    a100 = reference_registry.import_decode_schedule("llama-3.2-1b", "A100", 1)
    assert a100.package_name.endswith("A100.single_batch.decode_schedule") and a100.scheduler is not None
    with pytest.raises(NotImplementedError):
        reference_registry.decode_schedule_package_name("llama-3.2-1b", "B200", 65)
    with pytest.raises(NotImplementedError):
        reference_registry.decode_schedule_package_name("llama-3.2-1b", "A100", 17)
    with pytest.raises(NotImplementedError):
        reference_registry.decode_schedule_package_name("qwen2.5-3b", "B200", 1)
