"""ctypes binding of ``libjgb200.so``.

There is no fallback: if the library is missing or a call returns a status other
than ``JG_OK`` a ``RuntimeError`` is raised.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libjgb200.so")

_lib = None
_device_set = {}

vp = ctypes.c_void_p
i32 = ctypes.c_int32
i64 = ctypes.c_int64
sz = ctypes.c_size_t
f32 = ctypes.c_float

# name -> (restype, argtypes); one line per declaration in include/jgb200.h
SIGNATURES = {
    "jg_version": (ctypes.c_int, []),
    "jg_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "jg_last_error": (ctypes.c_char_p, []),
    "jg_set_device": (ctypes.c_int, [ctypes.c_int]),
    "jg_spmm_plan_bytes": (sz, [i64, i64, i32]),
    "jg_spmm_plan_build": (ctypes.c_int, [vp, i64, i64, i32, vp, sz, vp]),
    "jg_aggregate_workspace_bytes": (sz, [i64, i64, i64, i32]),
    "jg_aggregate_f32": (ctypes.c_int, [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp, i32, vp, sz, vp]),
    "jg_validate_segments": (ctypes.c_int, [vp, vp, i64, i64, i64, vp, sz, vp]),
    "jg_aggregate_add_f32": (ctypes.c_int, [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp, i32, vp, sz, vp]),
    "jg_aggregate_ordered_f32": (ctypes.c_int, [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp, i32, vp, sz, vp]),
    "jg_aggregate_bias_act_f32": (ctypes.c_int, [vp, vp, vp, vp, vp, vp, ctypes.c_int, i64, i64, i64, i64, vp, i32, vp, sz, vp]),
    "jg_aggregate_opts_f32": (ctypes.c_int, [vp, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                             i64, i64, i64, i64, vp, i32, vp, sz, vp]),
    "jg_halo_flag_bytes": (sz, []),
    "jg_halo_max_ranks": (ctypes.c_int, []),
    "jg_halo_flag_slots": (ctypes.c_int, []),
    "jg_halo_post": (ctypes.c_int, [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint32, vp]),
    "jg_halo_wait": (ctypes.c_int, [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint32, vp, i64, vp]),
    "jg_halo_pull": (ctypes.c_int, [vp, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, i64, ctypes.c_int, ctypes.c_uint32,
                                    vp, vp, i64, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp]),
    "jg_halo_pull_part": (ctypes.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, i64, ctypes.c_int,
                                         ctypes.c_uint32, vp, vp, i64, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp]),
    "jg_rows_to_half": (ctypes.c_int, [vp, vp, i64, vp]),
    "jg_partition_split_workspace_bytes": (sz, [i64]),
    "jg_partition_split": (ctypes.c_int, [vp, vp, vp, i64, i64, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "jg_halo_map_workspace_bytes": (sz, [i64]),
    "jg_halo_map_build": (ctypes.c_int, [vp, i64, i64, i32, i32, i32, vp, vp, vp, vp, sz, vp]),
    "jg_gather_rows_f32": (ctypes.c_int, [vp, vp, vp, i64, i64, i32, vp]),
    "jg_convert_workspace_bytes": (sz, [i64, i64]),
    "jg_coo_to_compressed": (ctypes.c_int, [vp, vp, i64, i64, ctypes.c_int, ctypes.c_int, vp, vp, vp, vp, sz, vp]),
    "jg_gcn_norm_compressed": (ctypes.c_int, [vp, vp, i64, i64, f32, ctypes.c_int, ctypes.c_int, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "jg_gcn_norm_coo_workspace_bytes": (sz, [i64, i64]),
    "jg_gcn_norm_coo": (ctypes.c_int, [vp, vp, i64, i64, f32, ctypes.c_int, vp, vp, vp, vp, vp, sz, vp]),
    "jg_to_undirected_workspace_bytes": (sz, [i64, i64]),
    "jg_to_undirected": (ctypes.c_int, [vp, vp, i64, i64, vp, vp, vp, vp, vp, sz, vp]),
    "jg_scatter_to_edge_f32": (ctypes.c_int, [vp, vp, vp, vp, i64, i64, i64, ctypes.c_int, vp]),
    "jg_edge_to_vertex_f32": (ctypes.c_int, [vp, vp, vp, vp, i64, i64, i64, ctypes.c_int, vp]),
    "jg_edge_softmax_fwd_f32": (ctypes.c_int, [vp, vp, vp, i64, i64, i64, vp]),
    "jg_edge_softmax_bwd_f32": (ctypes.c_int, [vp, vp, vp, vp, i64, i64, i64, vp]),
    "jg_gat_aggregate_workspace_bytes": (sz, [i64, i64, i64, i64]),
    "jg_gat_aggregate_supported": (ctypes.c_int, [i64, i64]),
    "jg_gat_plan_bytes": (sz, [i64]),
    "jg_gat_plan_build": (ctypes.c_int, [vp, i64, vp, sz, vp]),
    "jg_gat_aggregate_f32": (ctypes.c_int, [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, f32, vp, vp, sz, vp]),
    "jg_gat_backward_workspace_bytes": (sz, [i64, i64, i64, i64]),
    "jg_gat_backward_f32": (ctypes.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, f32, vp, vp, vp, sz, vp]),
    "jg_sample_counts_workspace_bytes": (sz, [i64]),
    "jg_sample_counts": (ctypes.c_int, [vp, i64, vp, i32, ctypes.c_int, vp, vp, sz, vp]),
    "jg_sample_neighbors": (ctypes.c_int, [vp, i64, vp, vp, vp, i32, ctypes.c_uint64, vp, i64, vp, vp]),
    "jg_expand_columns": (ctypes.c_int, [vp, i64, vp, vp, vp]),
    "jg_csc_to_csr_workspace_bytes": (sz, [i64, i64, i64]),
    "jg_csc_to_csr": (ctypes.c_int, [vp, vp, i64, i64, vp, vp, i64, i64, vp, vp, vp, vp, sz, vp]),
    "jg_degree_weights_workspace_bytes": (sz, [i64]),
    "jg_degree_weights": (ctypes.c_int, [i64, vp, i64, vp, vp, i64, vp, vp, sz, vp]),
    "jg_gemm_tf32_supported": (ctypes.c_int, [i64, i64, i64]),
    "jg_gemm_tf32_workspace_bytes": (sz, []),
    "jg_gemm_tf32": (ctypes.c_int, [vp, vp, vp, vp, i64, i64, i64, ctypes.c_int, vp, sz, vp]),
    "jg_gemm_tf32_dual": (ctypes.c_int, [vp, vp, vp, vp, vp, i64, i64, i64, ctypes.c_int, vp, sz, vp]),
    "jg_gemm_tf32_status": (ctypes.c_int, [vp, vp]),
    "jg_gemm_tf32_timeout_selftest": (ctypes.c_int, [vp, vp, vp, i64, i64, i64, ctypes.c_int32, ctypes.c_uint32, vp, sz, vp]),
    "jg_gemm_tn_tf32_supported": (ctypes.c_int, [i64, i64, i64]),
    "jg_gemm_tn_tf32_workspace_bytes": (sz, [i64, i64, i64]),
    "jg_gemm_tn_tf32": (ctypes.c_int, [vp, vp, vp, i64, i64, i64, vp, vp, sz, vp]),
    "jg_gemm_f32_workspace_bytes": (sz, [i64, i64, i64]),
    "jg_gemm_f32": (ctypes.c_int, [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, ctypes.c_int, vp, sz, vp]),
    "jg_aggregate_static_capacity_bytes": (sz, []),
    "jg_aggregate_f32_static": (ctypes.c_int, [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp]),
}


def lib():
    """The loaded library (loads on first use; raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m jittorgeometric_b200._build` "
                "(there is no CPU or eager fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status, what):
    if status != 0:
        L = lib()
        raise RuntimeError(f"{what}: {L.jg_status_string(status).decode()} "
                           f"[{status}] {L.jg_last_error().decode()}")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_for(t):
    """Current torch stream of the tensor's device, after making that device
    current for the library's own CUDA runtime on this thread."""
    if not t.is_cuda:
        raise RuntimeError("jittorgeometric_b200 operators need CUDA tensors (no CPU path exists)")
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    import threading
    key = threading.get_ident()
    if _device_set.get(key) != dev:
        check(lib().jg_set_device(dev), "jg_set_device")
        _device_set[key] = dev
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def workspace(nbytes, device):
    """Caller-owned scratch from torch's caching allocator."""
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
