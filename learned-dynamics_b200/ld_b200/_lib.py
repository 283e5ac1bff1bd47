"""ctypes binding of libld_hotpath.so. There is no fallback: if the library is missing or a call
fails, an exception is raised."""
import ctypes
import os

import torch

from .build import LIB_PATH

c_void_p, c_int, c_float, c_size_t, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_longlong

LD_OK, LD_ERR_SHAPE, LD_ERR_CAPACITY, LD_ERR_BOX_TOO_SMALL = 0, -1, -2, -3
LD_ERR_NONFINITE, LD_ERR_TIMEOUT, LD_ERR_CUDA, LD_ERR_WORKSPACE, LD_ERR_UNSUPPORTED = -4, -5, -6, -7, -8
LD_FLAG_CAPACITY, LD_FLAG_NONFINITE, LD_FLAG_TIMEOUT, LD_FLAG_OVERFLOW = 1, 2, 4, 8

# name -> argtypes ; every entry point declared in include/ld_hotpath.h
P, I, F, LL, SZ = c_void_p, c_int, c_float, c_ll, c_size_t
SIGNATURES = {
    "ld_radius_graph_workspace_size": [I, I, I, F, P, I, I, P],
    "ld_radius_graph_count": [P, I, I, I, F, P, I, I, P, SZ, P, P, P, P],
    "ld_radius_graph_fill": [P, I, I, I, F, P, I, I, P, SZ, P, LL, P, P, P, P, P, P],
    "ld_radius_graph_build_noalloc": [P, I, I, I, F, P, I, I, P, P, LL, P, P, P, P, P, P],
    "ld_row_ptr_from_sorted": [P, I, LL, I, P, P],
    "ld_segment_sum": [P, P, I, I, P, P],
    "ld_gather_rows": [P, P, I, LL, I, P, P],
    "ld_neighbour_lists_from_csr": [P, P, I, I, I, P, P, P, P],
    "ld_edges_read_padded": [P, P, P, I, I, I, I, P, P],
    "ld_edges_reduce_padded": [P, P, I, I, I, I, P, P],
    "ld_tensor_linear": [I, P, LL, LL, P, P, LL, I, I, P],
    "ld_tensor_linear_dw_workspace": [I, LL, I, I, P],
    "ld_tensor_linear_dw": [I, P, P, P, LL, I, I, P, SZ, P],
    "ld_bee_fwd": [P, P, P, P, P, P, LL, I, P, P],
    "ld_bee_self_products": [P, P, P, LL, I, P, P, P, I, P],
    "ld_linear_bf16_tc_in16": [P, LL, I, I, P, P, I, I, P, P, P],
    "ld_linear_bf16_tc_in16_res": [P, P, LL, I, I, P, P, I, I, P, P, P],
    "ld_bee_bw": [I, P, P, P, P, LL, I, P, P, P, P],
    "ld_cow_o0_fwd": [P, P, P, P, LL, I, P, P, P],
    "ld_cow_o0_bw": [P, P, P, P, LL, I, P, P, P],
    "ld_cow_o1_fwd": [P, P, P, P, LL, I, P, P, P, P],
    "ld_cow_o1_bw": [I, P, P, P, P, P, LL, I, P, P, P],
    "ld_mlp3_rows": [P, LL, I, P, P, I, P, P, I, P, P, I, I, P, P, P],
    "ld_pack_weights_bf16": [P, LL, LL, I, I, P, P],
    "ld_linear_bf16_tc": [P, LL, I, I, P, P, I, I, P, P, P],
    "ld_linear_bf16_tc_out16": [P, LL, I, I, P, P, I, I, P, LL, LL, I, P, P],
    "ld_linear_bf16_tc_out16_split": [P, LL, I, I, P, P, I, I, P, LL, LL, I, I, LL, I, P, P],
    "ld_group_norm_cm": [P, I, I, I, I, I, I, F, P, P, P, P, P],
    "ld_bee_self_products_cm": [P, P, P, LL, I, P, P, P, P],
    "ld_bee_messages_fused_bf16_tc": [P, P, P, I, I, I, F, P, P, P, P, P, P, P, P, P, P, P, F, P, P, P, P, P],
    "ld_bee_gamma_table": [P],
    "ld_painn_message_bf16_tc": [P, P, P, I, I, I, I, F, F, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P],
    "ld_painn_pack_gather": [P, P, I, I, P, P],
    "ld_radial_encode": [I, P, LL, I, F, P, P, P],
    "ld_linear_bf16_tc_selftest_timeout": [P, LL, I, P, I, P, P, P],
    "ld_counter_noise": [P, P, F, LL, LL, ctypes.c_ulonglong, ctypes.c_ulonglong, P],
    "ld_group_norm": [P, I, I, I, I, I, I, F, P, P, P, P, P],
    "ld_group_norm_res": [P, P, I, I, I, I, I, I, F, P, P, P, P, P],
    "ld_proxattn_fwd": [P, P, P, P, P, P, I, I, I, I, I, F, F, F, P, P],
    "ld_proxattn_fwd_tf32_tc": [P, P, P, P, P, P, I, I, I, I, I, F, F, F, P, P, P],
    "ld_proxattn_bwd": [P, P, P, P, P, P, I, I, I, I, I, F, F, F, P, P, P, P, P, P, P],
    "ld_ant16_contract_left": [I, P, P, LL, I, I, P, I, P],
    "ld_ant16_expand": [I, P, P, LL, I, I, P, P],
    "ld_ant16_contract_out": [I, P, P, LL, I, I, P, P],
    "ld_tensor_prod_bare": [I, I, I, I, P, P, LL, P, P],
    "ld_bee_messages_scalar_bf16_tc": [P, P, P, I, I, I, F, P, P, P, P, P, P, P, P, P, P, P, P, P, F, P, I, P, P],
    "ld_bee_messages_vd_f32": [P, P, P, I, I, F, P, P, P, P, P, P, F, P, P, I, I, P],
    "ld_bee_self_front_bf16_tc": [P, P, P, LL, I, I, I, I, P, P, P, P, P, P, P, P],
    "ld_bee_left_rows_bf16_tc": [P, P, P, LL, I, I, I, I, P, P, P, P, P, P],
    "ld_bee_messages_vd_bf16_tc": [P, P, P, I, I, F, P, P, P, P, F, P, P, P, P],
    "ld_bee_messages_scalar_f32": [P, P, P, I, I, I, F, P, P, P, P, P, P, P, P, P, P, P, P, P, P, F, P, P],
    "ld_painn_message_f32": [P, P, P, I, I, I, I, F, F, P, P, P, P, P, P, P, P, P, P, P, P, P, P],
}

_lib = None


class HotpathError(RuntimeError):
    def __init__(self, status, text):
        super().__init__(text)
        self.status = status


def lib():
    """The loaded shared library (loaded once). Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ld_b200.build` (needs nvcc); there is no CPU fallback")
        L = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        L.ld_packed_weight_elems.restype = c_ll
        L.ld_packed_weight_elems.argtypes = [c_int, c_int]
        L.ld_last_error.restype = ctypes.c_char_p
        L.ld_status_string.restype = ctypes.c_char_p
        L.ld_status_string.argtypes = [c_int]
        _lib = L
    return _lib


def check(status):
    if status != LD_OK:
        L = lib()
        detail = L.ld_last_error().decode() if status in (LD_ERR_CUDA, LD_ERR_SHAPE, LD_ERR_UNSUPPORTED, LD_ERR_BOX_TOO_SMALL, LD_ERR_WORKSPACE) else ""
        text = L.ld_status_string(status).decode()
        raise HotpathError(status, f"{text}: {detail}" if detail else text)


def ptr(t):
    """Device address of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr(device=None):
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda_f32(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32")


class KernelTimer:
    """Counts this library's kernel launches and, when enabled, times them with CUDA events
    recorded on the launching stream (used by bench.py for the per-kernel roofline)."""

    def __init__(self):
        self.reset(False)

    def reset(self, enabled=False):
        self.enabled = enabled
        self.pairs = {}
        self.launch_counts = {}
        self.total_launches = 0

    class _Region:
        def __init__(self, timer, name, launches):
            self.t, self.name, self.launches = timer, name, launches

        def __enter__(self):
            t = self.t
            t.total_launches += self.launches
            t.launch_counts[self.name] = t.launch_counts.get(self.name, 0) + self.launches
            if t.enabled:
                self.e0 = torch.cuda.Event(enable_timing=True)
                self.e1 = torch.cuda.Event(enable_timing=True)
                self.e0.record()
            return self

        def __exit__(self, *exc):
            if self.t.enabled:
                self.e1.record()
                self.t.pairs.setdefault(self.name, []).append((self.e0, self.e1))
            return False

    def region(self, name, launches=1):
        return KernelTimer._Region(self, name, launches)

    def summary(self):
        """name -> {launches, ms}; call after a device synchronize."""
        out = {}
        for name, pairs in self.pairs.items():
            out[name] = {"launches": len(pairs), "ms": sum(a.elapsed_time(b) for a, b in pairs)}
        return out


KERNEL_TIMER = KernelTimer()
