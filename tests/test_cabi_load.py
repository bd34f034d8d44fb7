"""CPU checks of the C ABI: the library loads without a driver, exports every symbol the header declares, and
rejects bad arguments on the host before anything is launched."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "momoe_b200.h")


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__
    __graft_entry__.build()
    from momoe import _lib
    return _lib


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(momoe_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported(lib):
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib.lib, n), "missing export " + n
    assert set(names) == set(lib.EXPORTED)


def test_capacity_arithmetic(lib):
    assert lib.lib.momoe_version() >= 100
    # 16384 tokens, 8 experts each, 128 experts: 1024 full tiles + one partial tile per expert at most
    assert lib.lib.momoe_tile_capacity(16384, 8, 128) == 1024 + 128
    assert lib.lib.momoe_sorted_rows_capacity(16384, 8, 128) == (1024 + 128) * 128
    assert lib.lib.momoe_sorted_rows_capacity(1, 8, 128) == (1 + 128) * 128
    assert lib.lib.momoe_permutation_workspace_bytes(16384, 128, 8) == (16384 // 64) * 128 * 4
    # small batches are permuted by one thread block, large ones by three kernels
    assert lib.lib.momoe_permutation_launches(64, 128, 8) == 1
    assert lib.lib.momoe_permutation_launches(1024, 256, 8) == 1
    assert lib.lib.momoe_permutation_launches(1025, 128, 8) == 3
    assert lib.lib.momoe_permutation_launches(64, 257, 8) == 3


def test_bad_arguments_rejected_on_host(lib):
    L = lib.lib
    assert L.momoe_route_topk(None, None, 4, 8, 2, 0, None, None, None, None, None, None, None, None) == -1
    one = C.c_void_p(16)  # never dereferenced: the calls below fail validation first
    assert L.momoe_route_topk(one, one, 4, 2048, 2, 0, one, one, None, None, None, None, None, None) == -4
    assert L.momoe_route_topk(one, one, 4, 8, 2, 2, one, one, None, None, None, None, None, None) == -1
    assert L.momoe_topk_from_mask(None, 1, 1, None, 1, 1, 4, 8, 2, None, None, None, None) == -1
    plan = lib.Plan(M=4, N=8, K=2, D=60, H=32, reserved=0, rows_capacity=128 * 9, sched=16, tile_expert=16,
                    pad_off=16, row_token=16, row_weight=16, pos_MK=16, status=16, pair_info=16)
    assert L.momoe_up_swiglu(C.byref(plan), one, one, one, None, None, 0, None) == -2   # D not a multiple of 8
    plan.D = 64
    assert L.momoe_up_swiglu(C.byref(plan), one, one, None, None, None, 0, None) == -1  # h missing
    assert L.momoe_up_swiglu(C.byref(plan), one, one, one, None, None, 1, None) == -1   # save buffers missing
    assert L.momoe_wgrad(C.byref(plan), one, 60, one, 64, one, None) == -2
    assert L.momoe_gather_rows(C.byref(plan), one, 60, one, None) == -2
    assert L.momoe_combine_rows(None, one, 64, one, None) == -1


def test_package_surface(lib):
    import inspect
    import momoe
    assert momoe.__all__ == ["MoMoE", "MoE", "TopKRouter"]
    assert list(inspect.signature(momoe.MoMoE.__init__).parameters)[1:] == [
        "embedding_dim", "intermediate_dim", "num_experts", "num_chosen_experts", "save_percent", "Wl1_ND2H",
        "Wl2_NHD"]
    assert list(inspect.signature(momoe.TopKRouter.__init__).parameters)[1:] == [
        "embedding_dim", "num_experts", "num_chosen_experts", "num_shared_experts", "Wg_DN"]
    assert list(inspect.signature(momoe.MoE.__init__).parameters)[1:] == [
        "embedding_dim", "intermediate_dim", "num_experts", "num_chosen_experts", "num_shared_experts",
        "save_percent", "bias_update_rate", "Wg_DN", "Wl1_ND2H", "Wl2_NHD"]


def test_modules_construct_on_cpu_but_refuse_to_run(lib):
    """Parameters can be built anywhere (state_dict keys as in the reference); running needs the GPU kernels."""
    import torch
    import momoe
    m = momoe.MoMoE(16, 8, 4, 2, 0, torch.zeros(4, 16, 16), torch.zeros(4, 8, 16))
    assert sorted(m.state_dict()) == ["Wl1_ND2H", "Wl2_NHD"]
    assert m.Wl1_ND2H.dtype == torch.bfloat16
    with pytest.raises(AssertionError):
        momoe.MoMoE(16, 8, 4, 2, 101, torch.zeros(4, 16, 16), torch.zeros(4, 8, 16))
    mask = torch.ones(4, 3, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(torch.zeros(1, 3, 16), mask, torch.ones(4, 3))
