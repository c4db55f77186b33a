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


def test_bench_layouts_and_cli():
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(os.path.dirname(os.path.dirname(__file__)),
                                                                            "bench.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    assert b.layout_for(1) == (1, 1, None, 1) and b.layout_for(2) == (2, 1, None, 1)
    assert b.layout_for(4) == (4, 1, None, 1) and b.layout_for(8) == (4, 2, 2, 1)      # the headline: TP4 x PP2, 2 virtual
    assert b.layout_for(8, "gpt3-1.3b") == (2, 1, None, 1) and b.layout_for(8, "mixtral") == (1, 1, None, 8)
    m = b.MODELS["llama7b"]
    assert (m["num_layers"], m["hidden_size"], m["ffn_hidden_size"], m["seq_length"], m["global_batch_size"]) == \
        (32, 4096, 11008, 4096, 64)
