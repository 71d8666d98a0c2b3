"""The reference's OWN host-side tests for this path, run against this package.

Where a checkout of the reference is at hand (BITMTP_REFERENCE, or a `reference` directory beside this
repository), its test modules for the runtime contracts are loaded from where they lie and executed with
`bonsai_sft.gpu.<module>` resolved to `bitmtp_b200.<module>`: option validation and role / width schedules of the
CLI, the kernel-shape registry, the strict-verification rules, the width selector, tokenizer / artifact
preflight, runtime profiles, release scope, the converter's input checks, and the evaluation driver's routing
checks (every recipe's widths and head precision reach the adapter; the keywords the adapter passes to the
decode loops exist in this package's signatures).  Nothing of the reference is copied;
without a checkout the module is skipped.  The methods listed in NOT_APPLICABLE are left out, each with its reason.
"""
import importlib
import importlib.util
import os
import sys
import types
import unittest

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("BITMTP_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
REF_TESTS = os.path.join(REF, "tests")

MODULES = ("test_bonsai_d4", "test_bonsai_strict_verifier", "test_bonsai_contracts",
           "test_generation_artifact_preflight", "test_orin_runtime", "test_bonsai_release_scope", "test_bonsai_cpu",
           "test_bonsai_converter", "test_evaluation_platforms")
MIRRORED = ("contracts", "run_generation", "fast_generate", "fast_runtime", "runtime_config", "model", "generate",
            "convert_bonsai_mtp_to_gpu", "checkpoint_validation")

NOT_APPLICABLE = {
    # acceptance is computed by a kernel here; these call it on host tensors / through the eager decoder
    "test_bonsai_strict_verifier.test_tied_logits_do_not_admit_a_different_token_id": "accept rule runs on the device",
    "test_bonsai_strict_verifier.test_acceptance_uses_only_ids_and_longest_prefix": "accept rule runs on the device",
    "test_bonsai_strict_verifier.test_eager_verifier_also_uses_ids_with_ties": "uncaptured eager decoders are out of scope",
    # nothing is traced or compiled here, and the only device is sm_100a
    "test_orin_runtime.test_orin_imports_and_eager_predicates_in_clean_process": "imports bonsai_sft in a child process",
    "test_orin_runtime.test_standard_delegates_without_changing_kwargs": "compile_helper is the identity",
    "test_orin_runtime.test_geometry_and_device_reject_unsupported_scope": "device rule is sm_100a",
    "test_bonsai_release_scope.test_4b_gpu_scope_requires_sm90": "device rule is sm_100a",
    "test_bonsai_release_scope.test_4b_q1_and_unknown_dimensions_are_rejected": "the padded vocabulary 151936 of synthetic checkpoints is accepted",
    # masks are a 16-byte step record here (their parity is pinned by the 308 recorded mask tensors)
    "test_bonsai_cpu.test_verifier_anchor_is_not_counted_twice": "additive mask tensors do not exist",
    "test_bonsai_cpu.test_ar_keeps_last_history_slot": "additive mask tensors do not exist",
    "test_bonsai_cpu.test_public_4b_guard_precedes_cuda_or_library_load": "every 1 <= M <= 32 is served; the registry check is opt-in",
    "test_bonsai_converter.test_valid_q1_synthetic_conversion_preserves_dtypes": "T2-g128 only",
    # the evaluation driver's own preflight wants lm-eval installed
    "test_evaluation_platforms.test_check_only_never_initializes_runtime_or_cuda": "lm-eval is not installed here",
}

pytestmark = pytest.mark.skipif(not os.path.isdir(REF_TESTS), reason="no checkout of the reference at hand")


@pytest.fixture(scope="module")
def aliased():
    """`bonsai_sft.gpu.*` -> `bitmtp_b200.*` for the duration of this module."""
    saved = {k: v for k, v in sys.modules.items() if k.split(".")[0] in ("bonsai_sft", "benchmarks")}
    for k in saved:
        del sys.modules[k]
    saved_path = list(sys.path)
    sys.path.insert(0, REF)                    # the reference's `benchmarks` package (its evaluation adapter and driver)
    pkg, gpu = types.ModuleType("bonsai_sft"), types.ModuleType("bonsai_sft.gpu")
    pkg.__path__, gpu.__path__ = [], []
    pkg.gpu = gpu
    sys.modules["bonsai_sft"], sys.modules["bonsai_sft.gpu"] = pkg, gpu
    for name in MIRRORED:
        mod = importlib.import_module("bitmtp_b200." + name)
        sys.modules["bonsai_sft.gpu." + name] = mod
        setattr(gpu, name, mod)
    yield
    for k in [k for k in sys.modules if k.split(".")[0] in ("bonsai_sft", "benchmarks")]:
        del sys.modules[k]
    sys.modules.update(saved)
    sys.path[:] = saved_path


def _cases(module_name):
    spec = importlib.util.spec_from_file_location("reference_" + module_name, os.path.join(REF_TESTS, module_name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    stack = [unittest.TestLoader().loadTestsFromModule(mod)]
    while stack:
        for t in stack.pop():
            if isinstance(t, unittest.TestSuite):
                stack.append(t)
            else:
                yield t


@pytest.mark.parametrize("module_name", MODULES)
def test_reference_host_tests_pass_against_this_package(aliased, module_name):
    ran, failed = 0, []
    cwd = os.getcwd()
    try:
        for case in _cases(module_name):
            key = f"{module_name}.{case._testMethodName}"
            if key in NOT_APPLICABLE:
                continue
            result = unittest.TestResult()
            case.run(result)
            ran += 1
            for _, trace in result.failures + result.errors:
                failed.append(f"{key}: {trace.strip().splitlines()[-1][:200]}")
    finally:
        os.chdir(cwd)
    assert not failed, "\n".join(failed)
    assert ran >= 3, f"{module_name}: only {ran} of the reference's tests ran"
