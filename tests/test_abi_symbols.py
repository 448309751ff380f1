"""The C-ABI library loads without a GPU and exports every entry point include/ling_b200.h declares."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ling_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ling_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_step_entry_points():
    names = declared_functions()
    for must in ("ling_b200_create", "ling_b200_verify_step", "ling_b200_kv_table_set", "ling_b200_describe_tree",
                 "ling_b200_kvpool_ensure", "ling_b200_select_batch", "ling_b200_start_plan"):
        assert must in names
    assert len(names) >= 60


def test_library_exports_every_declared_symbol(lb):
    L = lb.lib()
    missing = [n for n in declared_functions() if not hasattr(L, n)]
    assert not missing, missing


def test_abi_version_and_no_cpu_path(lb):
    assert lb.lib().ling_b200_abi_version() == 1
    # Without a GPU the compute entry points refuse loudly instead of falling back to a CPU path.
    if lb.lib().ling_b200_device_count() == 0:
        import numpy as np
        import pytest
        with pytest.raises(lb.LingError):
            lb.gemm_fp8(np.zeros((1, 128), np.float32), np.zeros((128, 128), np.float32))
        with pytest.raises(lb.LingError):
            lb.Context(lb.toy_config())
