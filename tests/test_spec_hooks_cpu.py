"""The backend-specialisation hooks (python/triton/runtime/driver.py:63-80) as the reference calls them, on CPU."""
import torch

from flagtree_b200 import spec


def test_ops_modify_all_appends_this_package_ops():
    # python/triton/ops/__init__.py:9-12: `__all__` goes through spec("ops_modify_all", __all__) and the result,
    # when truthy, replaces it
    names = ["matmul", "attention"]
    res = spec.ops_modify_all(names)
    assert res is names
    for op in ("sparse_mla_fwd", "sparse_mla_fwd_paged", "sparse_mla_merge", "kv_cache_write_fp8", "gemm_rs", "gemm_rs_fp8", "ag_gemm", "topk_indices"):
        assert op in res
    assert res[:2] == ["matmul", "attention"]
    import flagtree_b200
    for op in res[2:]:
        assert callable(getattr(flagtree_b200, op))


def test_matmul_hook_declines_what_it_does_not_handle():
    # a falsy return lets the reference's own kernel run (the convention of the hook)
    a = torch.zeros(8, 8, dtype=torch.float16)
    assert spec.matmul_kernel(None, a, a, a, 8, 8, 8, None, None, True, None) is None
    assert set(spec.__all__) == {"matmul_kernel", "ops_modify_all"}
