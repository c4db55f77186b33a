"""Every module of the package imports on a CPU-only machine (no GPU, no optional external libraries)."""
import importlib
import pkgutil

import megatron_lm_b200


def test_all_modules_import():
    failed = []
    for m in pkgutil.walk_packages(megatron_lm_b200.__path__, megatron_lm_b200.__name__ + "."):
        if m.name.endswith(("perf_test", "ec_bench", "report_memory", "preprocess_data", "merge_datasets", "microbench")):
            pass                                    # command-line modules import like any other
        try:
            importlib.import_module(m.name)
        except Exception as e:                      # noqa: BLE001
            failed.append((m.name, repr(e)[:200]))
    assert not failed, failed
