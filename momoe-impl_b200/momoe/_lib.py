"""ctypes binding of libmomoe_b200.so (the C ABI declared in include/momoe_b200.h).

There is no fallback: if the library is missing, importing this module raises with the build command.
"""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MOMOE_B200_LIB", os.path.join(_HERE, "libmomoe_b200.so"))

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "libmomoe_b200.so is not built; run `python momoe-impl_b200/build.py` (needs nvcc, targets sm_100a). "
        "There is no CPU or PyTorch fallback for the MoMoE kernels.")

lib = C.CDLL(LIB_PATH)

c_i32, c_i64, c_vp, c_sz, c_u32 = C.c_int32, C.c_int64, C.c_void_p, C.c_size_t, C.c_uint32


class Plan(C.Structure):
    """Mirror of momoe_plan_t."""
    _fields_ = [("M", c_i32), ("N", c_i32), ("K", c_i32), ("D", c_i32), ("H", c_i32), ("reserved", c_i32),
                ("rows_capacity", c_i64), ("sched", c_vp), ("tile_expert", c_vp), ("pad_off", c_vp),
                ("row_token", c_vp), ("row_weight", c_vp), ("pos_MK", c_vp), ("status", c_vp), ("pair_info", c_vp)]


PlanP = C.POINTER(Plan)

_PROTOS = {
    "momoe_version": (C.c_int, []),
    "momoe_sorted_rows_capacity": (c_i64, [c_i32, c_i32, c_i32]),
    "momoe_tile_capacity": (c_i64, [c_i32, c_i32, c_i32]),
    "momoe_route_topk": (C.c_int, [c_vp, c_vp, c_i32, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                                   c_vp]),
    "momoe_topk_from_mask": (C.c_int, [c_vp, c_i64, c_i64, c_vp, c_i64, c_i64, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp,
                                       c_vp]),
    "momoe_permutation_launches": (C.c_int, [c_i32, c_i32, c_i32]),
    "momoe_permutation_workspace_bytes": (c_sz, [c_i32, c_i32, c_i32]),
    "momoe_build_permutation": (C.c_int, [c_vp, c_vp, c_i32, c_i32, c_i32, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                                          c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_sz, c_vp, c_vp]),
    "momoe_build_permutation_static": (C.c_int, [c_vp, c_vp, c_i32, c_i32, c_i32, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp,
                                                 c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp]),
    "momoe_gather_rows": (C.c_int, [PlanP, c_vp, c_i32, c_vp, c_vp]),
    "momoe_combine_rows": (C.c_int, [PlanP, c_vp, c_i32, c_vp, c_vp]),
    "momoe_up_swiglu": (C.c_int, [PlanP, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp]),
    "momoe_up_swiglu_tokens": (C.c_int, [PlanP, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp]),
    "momoe_down_scale": (C.c_int, [PlanP, c_vp, c_vp, c_vp, c_vp]),
    "momoe_up_swiglu_decode": (C.c_int, [PlanP, c_vp, c_vp, c_vp, c_vp]),
    "momoe_down_scale_decode": (C.c_int, [PlanP, c_vp, c_vp, c_vp, c_vp]),
    "momoe_dgrad2_swiglu_bwd": (C.c_int, [PlanP, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "momoe_dgrad2_swiglu_bwd_tokens": (C.c_int, [PlanP, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "momoe_dgrad1": (C.c_int, [PlanP, c_vp, c_vp, c_vp, c_vp]),
    "momoe_wgrad": (C.c_int, [PlanP, c_vp, c_i32, c_vp, c_i32, c_vp, c_vp]),
    "momoe_wgrad_tokens": (C.c_int, [PlanP, c_vp, c_i32, c_i32, c_vp, c_i32, c_i32, c_vp, c_vp]),
    "momoe_scatter_gs": (C.c_int, [PlanP, c_vp, c_i32, c_vp, c_vp]),
    "momoe_router_backward": (C.c_int, [c_vp, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp,
                                        c_vp]),
    "momoe_router_backward_compact": (C.c_int, [c_vp, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp, c_vp]),
    "momoe_bias_update": (C.c_int, [c_vp, c_vp, c_i32, c_i32, C.c_float, C.c_float, c_vp]),
    "momoe_ep_set_wait_limit": (c_i64, [c_i64]),
    "momoe_ep_publish_counts": (C.c_int, [c_vp, c_i32, c_vp, c_vp, c_i32, c_i32, c_u32, c_vp, c_vp]),
    "momoe_ep_barrier": (C.c_int, [c_vp, c_i32, c_i32, c_u32, c_vp, c_vp]),
    "momoe_ep_plan": (C.c_int, [c_vp, c_i32, c_i32, c_i32, C.c_double, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                                c_vp, c_vp]),
    "momoe_ep_dispatch_rows": (C.c_int, [PlanP, c_vp, c_i32, c_vp, c_i32, c_vp, c_vp, c_vp, c_i32, c_i32, c_vp, c_vp,
                                         c_i32, c_vp]),
    "momoe_ep_combine_rows": (C.c_int, [PlanP, c_vp, c_vp, c_i32, c_i32, c_vp, c_i32, c_i32, c_vp]),
    "momoe_ep_plan_split": (C.c_int, [c_vp, c_i32, c_i32, c_i32, C.c_double, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                                      c_vp, c_i32, c_vp, c_vp, c_vp, c_vp]),
    "momoe_ep_dispatch_rows_range": (C.c_int, [PlanP, c_vp, c_i32, c_vp, c_i32, c_vp, c_vp, c_vp, c_i32, c_i32, c_vp,
                                               c_vp, c_i32, c_i32, c_i32, c_vp]),
    "momoe_ep_pull_rows": (C.c_int, [PlanP, c_vp, c_vp, c_i32, c_i32, c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, c_vp]),
    "momoe_ep_combine_rows_staged": (C.c_int, [PlanP, c_vp, c_vp, c_i32, c_i32, c_vp, c_i32, c_vp, c_i32, c_i32, c_i32,
                                               c_vp]),
    "momoe_ep_reduce_gs": (C.c_int, [c_vp, c_i32, c_vp, c_vp, c_vp]),
    "momoe_ep_pull_gs_compact": (C.c_int, [PlanP, c_vp, c_vp, c_i32, c_vp, c_i32, c_vp]),
}
for _name, (_res, _args) in _PROTOS.items():
    _f = getattr(lib, _name)
    _f.restype = _res
    _f.argtypes = _args

EXPORTED = tuple(_PROTOS)

_ERRORS = {-1: "bad argument (null pointer, size or alignment)", -2: "unsupported shape (D and H must be multiples "
           "of 8)", -3: "a CUDA call failed", -4: "exceeds a fixed capacity (N <= 1024, K <= 32)"}


def check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed: {_ERRORS.get(rc, 'code %d' % rc)}")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    if t is None:
        return None
    return C.c_void_p(t.data_ptr())


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("momoe (B200 build) runs on CUDA tensors only; there is no CPU path")
