"""Python face of the CUDA kernels: argument checks, then one C call per kernel.

Each function takes torch tensors that live on the GPU, checks device, dtype,
contiguity and the sizes the kernel takes, and launches on torch's current
stream.  A size a kernel refuses raises ``KernelSizeError`` with the kernel's name
and the offending numbers; nothing here falls back to torch or to the CPU.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Optional, Tuple

import torch

from .build import BuildError, build_library

F32, BF16 = 0, 1
STATUS_BITS = {
    1: "a token id outside the embedding table",
    2: "a page id outside the pool where a live position needs one",
    4: "a negative position or sequence index, or a position beyond the block table's row",
    8: "a row of logits without a comparable value (all NaN)",
    16: "a bounded wait inside a kernel ran out (the kernel gave up cleanly)",
}


class KernelError(RuntimeError):
    pass


class KernelSizeError(KernelError):
    pass


_lib = None
_lib_path = None
_lock = threading.Lock()

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_c_ll, _c_ull = ctypes.c_longlong, ctypes.c_ulonglong

_SIGNATURES = {
    "q3_embed": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_add_rmsnorm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "q3_add_rmsnorm_rows": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int,
                            _c_float, _c_void_p],
    "q3_rmsnorm": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "q3_gemm_f32_nt": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_rope_table": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p],
    "q3_qkv_post": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float,
                    _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p,
                    _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p],
    "q3_attn_ref": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                    _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                    _c_void_p, _c_void_p],
    "q3_attn_decode": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                       _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                       _c_void_p, _c_void_p],
    "q3_attn_decode_tma": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                           _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                           _c_void_p, _c_void_p],
    "q3_attn_decode_tma_qkv": [_c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                               _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                               _c_int, _c_float, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_attn_prefill": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p,
                        _c_void_p],
    "q3_attn_tc": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    "q3_swiglu": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_gemm_tc": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                   _c_void_p],
    "q3_gemm_tc_pair": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                        _c_void_p],
    "q3_gemm_tc_qkv": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float,
                       _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                       _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_gemm_skinny": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_gemm_skinny_fused": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                             _c_int, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "q3_sample": [_c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_ull, _c_int,
                  _c_void_p, _c_ll, _c_void_p, _c_void_p, _c_void_p],
    "q3_scale_add_rmsnorm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_float,
                             _c_void_p],
    "q3_gated_act": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_token_shift": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                       _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_causal_conv": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                       _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_block_diag": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_rglru_scan": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                      _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                      _c_int, _c_void_p, _c_void_p],
    "q3_rglru_scan_chunked": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                              _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                              _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_selective_scan_chunked": [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                  _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                                  _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_selective_scan": [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                          _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_void_p, _c_void_p],
    "q3_qk_gate_post": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float,
                        _c_float, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int,
                        _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p],
    "q3_attn_sigmoid_tc": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                           _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                           _c_void_p, _c_void_p],
    "q3_attn_sigmoid_mma": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                            _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                            _c_float, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_attn_sigmoid": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                        _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                        _c_void_p, _c_void_p],
    "q3_embed_scaled": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p,
                        _c_void_p],
    "q3_hc_norm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                   _c_int, _c_float, _c_void_p, _c_void_p],
    "q3_hc_sum_norm_rows": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                            _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    "q3_softcap": [_c_void_p, _c_ll, _c_float, _c_void_p],
    "q3_act": [_c_void_p, _c_void_p, _c_int, _c_ll, _c_int, _c_void_p],
    "q3_latent_kv_post": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                          _c_float, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                          _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_latent_q_post": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_void_p,
                         _c_int, _c_int, _c_int, _c_void_p],
    "q3_latent_attn_ref": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                           _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p,
                           _c_void_p],
    "q3_latent_attn_mma": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                           _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                           _c_void_p, _c_void_p, _c_void_p],
    "q3_gate_heads": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_ssd_scan": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                    _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                    _c_int, _c_void_p, _c_void_p],
    "q3_ssd_scan_mma": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                        _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                        _c_void_p],
    "q3_gated_group_norm": [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                            _c_float, _c_void_p],
    "q3_add_layernorm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int,
                         _c_float, _c_void_p],
    "q3_add_layernorm_conv1": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                               _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    "q3_stream_concat": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "q3_input_conv": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                      _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_pw_qkv_post": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float,
                       _c_int, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p,
                       _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_pool_blocks": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                       _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                       _c_void_p, _c_void_p],
    "q3_pw_attn_ref": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                       _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_float, _c_int, _c_void_p, _c_void_p],
    "q3_pw_attn_mma": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p,
                       _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_float, _c_float, _c_float, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                       _c_ll, _c_void_p, _c_void_p],
    "q3_mingru_scan": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                       _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p, _c_void_p],
    "q3_moe_grouped": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                       _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_void_p, _c_void_p, _c_void_p],
    "q3_mingru_scan_chunked": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                               _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                               _c_float, _c_void_p, _c_void_p],
    "q3_moe_route": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                     _c_float, _c_void_p],
    "q3_moe_pairs": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "q3_add_dyt": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                   _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_side_gate": [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "q3_add_unit_rms": [_c_void_p, _c_void_p, _c_void_p, _c_float, _c_int, _c_int, _c_int, _c_void_p],
    "q3_sigmoid_gate": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "q3_mlstm_scan": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float, _c_void_p,
                      _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                      _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "q3_mlstm_out": [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_float, _c_float, _c_void_p, _c_int, _c_int, _c_int,
                     _c_int, _c_int, _c_void_p],
}


_WAIT_TEST = ("q3_gemm_tc_wait_test", "q3_attn_tc_wait_test", "q3_attn_decode_tma_wait_test")


def library() -> ctypes.CDLL:
    """The loaded kernel library; compiles it at the first call if it is not built yet."""
    global _lib, _lib_path
    if _lib is None:
        with _lock:
            if _lib is None:
                try:
                    path = build_library()
                except BuildError as e:
                    raise KernelError(str(e)) from None
                lib = ctypes.CDLL(path)
                for name, argtypes in _SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.argtypes = argtypes
                    fn.restype = _c_int
                for name in _WAIT_TEST:
                    fn = getattr(lib, name)
                    fn.argtypes = [ctypes.c_uint, _c_int]
                    fn.restype = _c_int
                lib.q3_sm_count.argtypes = []
                lib.q3_sm_count.restype = _c_int
                lib.q3_attn_decode_blocks_per_sm.argtypes = [_c_int]
                lib.q3_attn_decode_blocks_per_sm.restype = _c_int
                lib.q3_latent_attn_mma_takes.argtypes = [_c_int, _c_int]
                lib.q3_latent_attn_mma_takes.restype = _c_int
                lib.q3_pw_attn_mma_takes.argtypes = [_c_int, _c_int]
                lib.q3_pw_attn_mma_takes.restype = _c_int
                lib.q3_ssd_record_floats.argtypes = [_c_int, _c_int, _c_int]
                lib.q3_ssd_record_floats.restype = _c_ll
                lib.q3_ssd_mma_takes.argtypes = [_c_int, _c_int]
                lib.q3_ssd_mma_takes.restype = _c_int
                lib.q3_ssd_mma_record_floats.argtypes = [_c_int, _c_int, _c_int]
                lib.q3_ssd_mma_record_floats.restype = _c_ll
                lib.q3_ssd_chunk.argtypes = []
                lib.q3_ssd_chunk.restype = _c_int
                lib.q3_scan_chunk.argtypes = []
                lib.q3_scan_chunk.restype = _c_int
                lib.q3_mingru_chunk.argtypes = []
                lib.q3_mingru_chunk.restype = _c_int
                lib.q3_mlstm_max_dim.argtypes = []
                lib.q3_mlstm_max_dim.restype = _c_int
                lib.q3_moe_tile_rows.argtypes = []
                lib.q3_moe_tile_rows.restype = _c_int
                lib.q3_sample_scratch_bytes.argtypes = [_c_int]
                lib.q3_sample_scratch_bytes.restype = _c_ll
                _lib, _lib_path = _Counting(lib), path
    return _lib


class _Counting:
    """The library with every launcher call counted (the benchmark reports launches per step)."""

    def __init__(self, lib):
        self._lib = lib
        self.calls = 0

    def __getattr__(self, name):
        if name not in _SIGNATURES:  # without declared argument types ctypes would cut pointers to 32 bits
            raise KernelError(f"{name}: no argument types declared for this entry point")
        fn = getattr(self._lib, name)

        def counted(*args):
            self.calls += 1
            return fn(*args)

        setattr(self, name, counted)
        return counted


def launch_count() -> int:
    """Kernel launches made through this module so far."""
    return library().calls


def library_path() -> Optional[str]:
    library()
    return _lib_path


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(name: str, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; the kernels run on the GPU only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous (shape {tuple(t.shape)}, strides {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")


def _done(kernel: str, code: int, detail: str = "") -> None:
    if code == 0:
        return
    if code == -2:
        raise KernelSizeError(f"{kernel}: size not taken by this kernel ({detail})")
    if code == -1:
        raise KernelError(f"{kernel}: dtype not taken ({detail})")
    if code == -3:
        raise KernelError(f"{kernel}: misaligned argument ({detail})")
    if code == -4:
        raise KernelSizeError(f"{kernel}: needs more scratch memory than is provided ({detail})")
    if code == -5:
        raise KernelError(f"{kernel}: the CUDA driver refused a tensor-map request ({detail})")
    raise KernelError(f"{kernel}: CUDA launch failed with error {code} ({detail})")


def set_wait_test(limit: int = 0, drop_copy: int = -1) -> None:
    """For tests of the path on which a kernel gives up a wait: every wait on an mbarrier in the TMA / tcgen05
    kernels polls ``limit`` times (0: the serving default of 2^24) and the loader of each leaves out its copy
    number ``drop_copy`` (-1: none), whose barrier then never completes.  Call it with no arguments to put the
    defaults back.  Synchronises the device."""
    torch.cuda.synchronize()
    for name in _WAIT_TEST:
        code = getattr(library()._lib, name)(int(limit), int(drop_copy))
        if code:
            raise KernelError(f"{name}: CUDA error {code}")
    torch.cuda.synchronize()


def describe_status(word: int) -> str:
    return "; ".join(text for bit, text in STATUS_BITS.items() if word & bit) or "ok"


# ------------------------------------------------------------------ kernels
def embed(table: torch.Tensor, ids: torch.Tensor, resid: torch.Tensor, status: torch.Tensor) -> None:
    """resid[t] = float32(table[ids[t]])."""
    _check("embed.table", table)
    _check("embed.ids", ids, torch.int32)
    _check("embed.resid", resid, torch.float32)
    T, H = resid.shape
    V = table.shape[0]
    if table.shape[1] != H or ids.numel() != T:
        raise KernelError(f"embed: table {tuple(table.shape)}, ids {tuple(ids.shape)}, resid {tuple(resid.shape)}")
    code = library().q3_embed(table.data_ptr(), dtype_tag(table.dtype), ids.data_ptr(), resid.data_ptr(),
                              T, H, V, status.data_ptr(), _stream())
    _done("embed", code)


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                out: torch.Tensor, eps: float) -> None:
    """resid += delta (when given); out = rmsnorm(resid) * weight."""
    _check("add_rmsnorm.resid", resid, torch.float32)
    _check("add_rmsnorm.weight", weight, torch.float32)
    _check("add_rmsnorm.out", out)
    T, H = resid.shape
    if delta is not None:
        _check("add_rmsnorm.delta", delta, out.dtype)
        if tuple(delta.shape) != (T, H):
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs stream {(T, H)}")
    if tuple(out.shape) != (T, H) or weight.numel() != H:
        raise KernelError(f"add_rmsnorm: out {tuple(out.shape)}, weight {tuple(weight.shape)}, stream {(T, H)}")
    code = library().q3_add_rmsnorm(resid.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(),
                                    dtype_tag(out.dtype), T, H, float(eps), _stream())
    _done("add_rmsnorm", code, f"width {H}")


def add_rmsnorm_rows(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                     rows: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out[r] = rmsnorm(resid[rows[r]] + delta[rows[r]]) * weight; resid is left as it is."""
    _check("add_rmsnorm_rows.resid", resid, torch.float32)
    _check("add_rmsnorm_rows.weight", weight, torch.float32)
    _check("add_rmsnorm_rows.rows", rows, torch.int32)
    _check("add_rmsnorm_rows.out", out)
    T, H = resid.shape
    R = rows.numel()
    if delta is not None:
        _check("add_rmsnorm_rows.delta", delta, out.dtype)
        if tuple(delta.shape) != (T, H):
            raise KernelError(f"add_rmsnorm_rows: delta {tuple(delta.shape)} vs stream {(T, H)}")
    if tuple(out.shape) != (R, H) or weight.numel() != H:
        raise KernelError(f"add_rmsnorm_rows: out {tuple(out.shape)}, rows {R}, width {H}")
    if R == 0:
        return
    code = library().q3_add_rmsnorm_rows(resid.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(),
                                         dtype_tag(out.dtype), rows.data_ptr(), R, H, float(eps), _stream())
    _done("add_rmsnorm_rows", code, f"width {H}")


def scale_add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                      out: Optional[torch.Tensor], alpha: float, eps: float) -> None:
    """resid = rmsnorm(alpha * resid + delta) * weight, in place in the float32 stream; ``out`` (optional) gets
    the same rows in its own dtype (the dtype of ``delta``)."""
    _check("scale_add_rmsnorm.resid", resid, torch.float32)
    _check("scale_add_rmsnorm.weight", weight, torch.float32)
    T, H = resid.shape
    dtype = None
    for name, t in (("delta", delta), ("out", out)):
        if t is not None:
            _check(f"scale_add_rmsnorm.{name}", t, dtype)
            dtype = t.dtype
            if tuple(t.shape) != (T, H):
                raise KernelError(f"scale_add_rmsnorm: {name} {tuple(t.shape)} vs stream {(T, H)}")
    if weight.numel() != H:
        raise KernelError(f"scale_add_rmsnorm: weight {tuple(weight.shape)}, stream {(T, H)}")
    code = library().q3_scale_add_rmsnorm(resid.data_ptr(), _ptr(delta), weight.data_ptr(), _ptr(out),
                                          dtype_tag(dtype or torch.float32), T, H, float(alpha), float(eps), _stream())
    _done("scale_add_rmsnorm", code, f"width {H}")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out[r] = rmsnorm(x[r]) * weight over the last dimension."""
    _check("rmsnorm.x", x)
    _check("rmsnorm.out", out, x.dtype)
    _check("rmsnorm.weight", weight, torch.float32)
    dim = x.shape[-1]
    rows = x.numel() // dim if dim else 0
    if out.shape != x.shape or weight.numel() != dim:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)}, out {tuple(out.shape)}, weight {tuple(weight.shape)}")
    code = library().q3_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_tag(x.dtype), rows, dim,
                                float(eps), _stream())
    _done("rmsnorm", code)


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in plain float32 (no tensor cores)."""
    _check("gemm_f32_nt.a", a, torch.float32)
    _check("gemm_f32_nt.w", w, torch.float32)
    _check("gemm_f32_nt.out", out, torch.float32)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_f32_nt: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    code = library().q3_gemm_f32_nt(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, K, K, N, _stream())
    _done("gemm_f32_nt", code, f"M {M} N {N} K {K}")


def qkv_post(qkv: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
             q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
             inv_freq: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
             tok_seq: torch.Tensor, block_table: torch.Tensor, num_q_heads: int, num_kv_heads: int,
             head_dim: int, write_kv: bool, status: torch.Tensor, cos_sin: Optional[torch.Tensor] = None) -> None:
    """Head norm, rotation, q to its buffer and k/v into their pages, in one pass over qkv.
    ``cos_sin``: the table of ``rope_table`` for the same positions and inv_freq (optional)."""
    _check("qkv_post.qkv", qkv)
    _check("qkv_post.q_out", q_out, qkv.dtype)
    _check("qkv_post.k_pages", k_pages, qkv.dtype)
    _check("qkv_post.v_pages", v_pages, qkv.dtype)
    _check("qkv_post.positions", positions, torch.int32)
    _check("qkv_post.tok_seq", tok_seq, torch.int32)
    _check("qkv_post.block_table", block_table, torch.int32)
    T = qkv.shape[0]
    width = (num_q_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width or q_out.numel() != T * num_q_heads * head_dim:
        raise KernelError(f"qkv_post: qkv {tuple(qkv.shape)} expected [T, {width}]; q_out {tuple(q_out.shape)}")
    num_pages, hkv, page_size, d = k_pages.shape
    if hkv != num_kv_heads or d != head_dim or v_pages.shape != k_pages.shape:
        raise KernelError(f"qkv_post: pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)} "
                          f"vs heads {num_kv_heads} x {head_dim}")
    if positions.numel() != T or tok_seq.numel() != T or block_table.dim() != 2:
        raise KernelError("qkv_post: positions / tok_seq must have one entry per token; block_table is 2-D")
    for name, wt in (("q_weight", q_weight), ("k_weight", k_weight)):
        if wt is not None:
            _check(f"qkv_post.{name}", wt, torch.float32)
            if wt.numel() != head_dim:
                raise KernelError(f"qkv_post: {name} has {wt.numel()} elements, head_dim is {head_dim}")
    if inv_freq is not None:
        _check("qkv_post.inv_freq", inv_freq, torch.float32)
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError(f"qkv_post: inv_freq has {inv_freq.numel()} entries, rotary_dim is {rotary_dim}")
    if cos_sin is not None:
        _check("qkv_post.cos_sin", cos_sin, torch.float32)
        if inv_freq is None or tuple(cos_sin.shape) != (T, rotary_dim):
            raise KernelError(f"qkv_post: cos_sin {tuple(cos_sin.shape)} expected [{T}, {rotary_dim}] with inv_freq")
    code = library().q3_qkv_post(
        qkv.data_ptr(), dtype_tag(qkv.dtype), T, num_q_heads, num_kv_heads, head_dim, _ptr(q_weight),
        _ptr(k_weight), float(eps), _ptr(inv_freq), _ptr(cos_sin), int(rotary_dim), positions.data_ptr(), tok_seq.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, k_pages.data_ptr(), v_pages.data_ptr(),
        num_pages, q_out.data_ptr(), 1 if write_kv else 0, status.data_ptr(), _stream())
    _done("qkv_post", code, f"head_dim {head_dim}, rotary_dim {rotary_dim}")


def rope_table(inv_freq: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> None:
    """table[t] = cos(positions[t] * inv_freq) then sin(...): float32 [T, 2 * len(inv_freq)]."""
    _check("rope_table.inv_freq", inv_freq, torch.float32)
    _check("rope_table.positions", positions, torch.int32)
    _check("rope_table.table", table, torch.float32)
    T, half = positions.numel(), inv_freq.numel()
    if tuple(table.shape) != (T, 2 * half):
        raise KernelError(f"rope_table: table {tuple(table.shape)} expected [{T}, {2 * half}]")
    code = library().q3_rope_table(inv_freq.data_ptr(), positions.data_ptr(), table.data_ptr(), T, half, _stream())
    _done("rope_table", code)


def attn_ref(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
             q_start: torch.Tensor, kv_len: torch.Tensor, tok_seq: torch.Tensor,
             block_table: torch.Tensor, scale: float, window: int, status: torch.Tensor) -> None:
    """Plain paged causal attention (one warp per query and head); any head_dim up to 512."""
    _check("attn_ref.q", q)
    _check("attn_ref.out", out, q.dtype)
    _check("attn_ref.k_pages", k_pages, q.dtype)
    _check("attn_ref.v_pages", v_pages, q.dtype)
    for name, t in (("q_start", q_start), ("kv_len", kv_len), ("tok_seq", tok_seq), ("block_table", block_table)):
        _check(f"attn_ref.{name}", t, torch.int32)
    T, Hq, D = q.shape
    num_pages, Hkv, page_size, d = k_pages.shape
    if d != D or v_pages.shape != k_pages.shape or out.numel() != q.numel():
        raise KernelError(f"attn_ref: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    code = library().q3_attn_ref(q.data_ptr(), dtype_tag(q.dtype), k_pages.data_ptr(), v_pages.data_ptr(),
                                 out.data_ptr(), q_start.data_ptr(), kv_len.data_ptr(), tok_seq.data_ptr(),
                                 block_table.data_ptr(), block_table.shape[1], page_size, num_pages, T, Hq, Hkv,
                                 D, float(scale), int(window), status.data_ptr(), _stream())
    _done("attn_ref", code, f"heads {Hq}/{Hkv}, head_dim {D}")


ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "none": 3, "relu_sq": 4}


def activation_code(name: str, gate: bool = False) -> int:
    if name not in ACTIVATIONS or (gate and name == "none"):
        raise KernelError(f"activation '{name}' is not built (built: {', '.join(ACTIVATIONS)})")
    return ACTIVATIONS[name]


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, interleave8: bool = False, activation: str = "silu") -> None:
    """out = up * act(gate); gate = first half of the columns and up = second half, or with
    ``interleave8`` alternating blocks of eight columns (gate, up, gate, up, ...)."""
    _check("gated_act.gate_up", gate_up)
    _check("gated_act.out", out, gate_up.dtype)
    T, two_i = gate_up.shape
    if two_i % 2 or tuple(out.shape) != (T, two_i // 2):
        raise KernelError(f"gated_act: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
    code = library().q3_gated_act(gate_up.data_ptr(), out.data_ptr(), dtype_tag(out.dtype), T, two_i // 2,
                                  1 if interleave8 else 0, activation_code(activation, gate=True), _stream())
    _done("gated_act", code, f"width {two_i // 2}")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleave8: bool = False) -> None:
    """``gated_act`` with the SiLU gate."""
    gated_act(gate_up, out, interleave8, "silu")


SKINNY_MAX_ROWS = 16  # rows of the few-rows product (two tiles of eight tokens)


def gemm_skinny_takes(rows: int, weight: torch.Tensor) -> bool:
    return rows <= SKINNY_MAX_ROWS and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu_blocks: bool = False,
                activation: str = "silu", plain_activation: Optional[str] = None) -> None:
    """out[T, N] = x[T, K] @ w[N, K]^T for T <= 16, bfloat16 in, out bfloat16 or float32.
    ``swiglu_blocks``: w's rows alternate gate/up in blocks of eight and out is [T, N / 2] = up * act(gate).
    ``plain_activation`` (without ``swiglu_blocks``): out = act(x w^T), the activation applied before the store."""
    _check("gemm_skinny.x", x, torch.bfloat16)
    _check("gemm_skinny.w", w, torch.bfloat16)
    _check("gemm_skinny.out", out)
    T, K = x.shape
    N = w.shape[0]
    want_cols = N // 2 if swiglu_blocks else N
    if w.shape[1] != K or tuple(out.shape) != (T, want_cols) or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_skinny: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    code = library().q3_gemm_skinny(x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, want_cols,
                                    1 if out.dtype == torch.float32 else 0,
                                    1 + activation_code(activation, gate=True) if swiglu_blocks else (
                                        -1 - activation_code(plain_activation, gate=True) if plain_activation else 0),
                                    _stream())
    _done("gemm_skinny", code, f"T {T} N {N} K {K}")


SUMSQ_ROWS = 16  # row pitch of the partial sums of squares that the fused few-rows products exchange


def sumsq_parts(features: int) -> int:
    """Partial sums per row that ``gemm_skinny_into_stream`` leaves for a stream ``features`` wide."""
    return (features + 15) // 16


def gemm_skinny_normed_pays(rows: int, weight: torch.Tensor) -> bool:
    """Whether a decode step without norm kernels is the faster one for this many rows and this reduction
    length: always with one token tile (up to 8 rows); with two only while the reduction is short, where the
    product with two token tiles is not yet short of registers (measured: profiles/decode_step_rules.md)."""
    return rows <= 8 or weight.shape[1] <= 3072


def gemm_skinny_normed(scaled: torch.Tensor, sumsq: torch.Tensor, parts: int, eps: float, w: torch.Tensor,
                       out: torch.Tensor, swiglu_blocks: bool = False) -> None:
    """out = rmsnorm(stream) @ w^T for up to 16 rows without a norm kernel.  ``scaled`` is the stream times
    the norm's weight in bfloat16 and ``sumsq[p, t]`` for ``p < parts`` are partial sums of squares of the
    stream's row ``t``, both as ``gemm_skinny_into_stream`` leaves them; the product of ``scaled`` is multiplied
    by the row's 1 / rms = 1 / sqrt(sum / K + eps) before it is stored.  ``swiglu_blocks`` as in ``gemm_skinny``."""
    _check("gemm_skinny_normed.scaled", scaled, torch.bfloat16)
    _check("gemm_skinny_normed.sumsq", sumsq, torch.float32)
    _check("gemm_skinny_normed.w", w, torch.bfloat16)
    _check("gemm_skinny_normed.out", out, torch.bfloat16)
    T, K = scaled.shape
    N = w.shape[0]
    want_cols = N // 2 if swiglu_blocks else N
    if (w.shape[1] != K or tuple(out.shape) != (T, want_cols) or sumsq.dim() != 2
            or sumsq.shape[1] != SUMSQ_ROWS or not 0 < parts <= sumsq.shape[0]):
        raise KernelError(f"gemm_skinny_normed: operand {tuple(scaled.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, "
                          f"sums {tuple(sumsq.shape)} of which {parts}")
    code = library().q3_gemm_skinny_fused(scaled.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, want_cols,
                                          4 if swiglu_blocks else 3, sumsq.data_ptr(), int(parts), float(eps), None, None,
                                          None, _stream())
    _done("gemm_skinny_normed", code, f"T {T} N {N} K {K}")


def gemm_skinny_into_stream(x: torch.Tensor, w: torch.Tensor, stream: torch.Tensor, sumsq: torch.Tensor,
                            next_weight: Optional[torch.Tensor] = None, scaled: Optional[torch.Tensor] = None) -> int:
    """stream += x @ w^T for up to 16 rows (x, w bfloat16; stream float32), and ``sumsq[p, t]`` = the sum of
    squares of the 16 new values ``stream[t, 16 p : 16 p + 16]``; returns the number of such parts.  With
    ``next_weight`` (the weight of the norm that comes next) and ``scaled`` (bfloat16, like stream):
    ``scaled = stream * next_weight``, rounded once: the operand of ``gemm_skinny_normed``."""
    _check("gemm_skinny_into_stream.x", x, torch.bfloat16)
    _check("gemm_skinny_into_stream.w", w, torch.bfloat16)
    _check("gemm_skinny_into_stream.stream", stream, torch.float32)
    _check("gemm_skinny_into_stream.sumsq", sumsq, torch.float32)
    T, K = x.shape
    N = w.shape[0]
    parts = sumsq_parts(N)
    if (w.shape[1] != K or tuple(stream.shape) != (T, N) or sumsq.dim() != 2 or sumsq.shape[1] != SUMSQ_ROWS
            or sumsq.shape[0] < parts or (next_weight is None) != (scaled is None)):
        raise KernelError(f"gemm_skinny_into_stream: x {tuple(x.shape)}, w {tuple(w.shape)}, stream "
                          f"{tuple(stream.shape)}, sums {tuple(sumsq.shape)}")
    if scaled is not None:
        _check("gemm_skinny_into_stream.next_weight", next_weight, torch.float32)
        _check("gemm_skinny_into_stream.scaled", scaled, torch.bfloat16)
        if next_weight.numel() != N or tuple(scaled.shape) != (T, N):
            raise KernelError(f"gemm_skinny_into_stream: next weight {tuple(next_weight.shape)}, scaled "
                              f"{tuple(scaled.shape)} for a stream {(T, N)}")
    code = library().q3_gemm_skinny_fused(x.data_ptr(), w.data_ptr(), stream.data_ptr(), T, N, K, N, 2, None, 0,
                                          0.0, sumsq.data_ptr(), _ptr(next_weight), _ptr(scaled), _stream())
    _done("gemm_skinny_into_stream", code, f"T {T} N {N} K {K}")
    return parts


def sample(logits: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
           temperature: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
           request_key: Optional[torch.Tensor] = None, position: Optional[torch.Tensor] = None,
           seed: int = 0) -> None:
    """One token per row of float32 logits: argmax where temperature <= 0, else a Gumbel-max draw
    (among the top_k largest logits where top_k > 0)."""
    _check("sample.logits", logits, torch.float32)
    _check("sample.out", out, torch.int32)
    R, V = logits.shape
    if out.numel() != R:
        raise KernelError(f"sample: {R} rows of logits, {out.numel()} outputs")
    if temperature is not None:
        _check("sample.temperature", temperature, torch.float32)
        if request_key is None or position is None:
            raise KernelError("sample: a temperature needs request_key and position")
        _check("sample.request_key", request_key, torch.int64)
        _check("sample.position", position, torch.int32)
    if top_k is not None:
        _check("sample.top_k", top_k, torch.int32)
    scratch = _sample_scratch(logits.device, R)
    code = library().q3_sample(logits.data_ptr(), R, V, V, _ptr(temperature), _ptr(top_k), _ptr(request_key),
                               _ptr(position), int(seed) & 0xFFFFFFFFFFFFFFFF,
                               1 if (top_k is not None and temperature is not None) else 0, scratch.data_ptr(),
                               scratch.numel(), out.data_ptr(), status.data_ptr(), _stream())
    _done("sample", code)


_SAMPLE_SCRATCH = {}


def _sample_scratch(device: torch.device, rows: int) -> torch.Tensor:
    """Zero-filled working memory of the sampling kernels for up to ``rows`` rows (they leave it zeroed)."""
    have = _SAMPLE_SCRATCH.get(device)
    need = int(library()._lib.q3_sample_scratch_bytes(max(rows, 8)))
    if have is None or have.numel() < need:
        have = torch.zeros(need, dtype=torch.uint8, device=device)
        _SAMPLE_SCRATCH[device] = have
    return have


def rope(x: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, positions: torch.Tensor,
         out: torch.Tensor, status: torch.Tensor) -> None:
    """out = rotate-half rotary encoding of x[T, heads, D] at `positions` (no norm, no cache)."""
    _check("rope.x", x)
    _check("rope.out", out, x.dtype)
    _check("rope.inv_freq", inv_freq, torch.float32)
    _check("rope.positions", positions, torch.int32)
    T, heads, d = x.shape
    if out.shape != x.shape or positions.numel() != T or inv_freq.numel() * 2 != rotary_dim:
        raise KernelError(f"rope: x {tuple(x.shape)}, out {tuple(out.shape)}, positions {positions.numel()}, "
                          f"inv_freq {inv_freq.numel()}, rotary_dim {rotary_dim}")
    code = library().q3_qkv_post(
        x.data_ptr(), dtype_tag(x.dtype), T, heads, 0, d, None, None, 0.0, inv_freq.data_ptr(), None, int(rotary_dim),
        positions.data_ptr(), positions.data_ptr(), None, 1, 1, None, None, 0, out.data_ptr(), 0,
        status.data_ptr(), _stream())
    _done("rope", code, f"head_dim {d}, rotary_dim {rotary_dim}")


def gemm_tc_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[1] % 8 == 0


def gemm_tc_swiglu_pays(rows: int, weight: torch.Tensor) -> Optional[str]:
    """Which of the engine's tcgen05 gate/up products with SwiGLU in the epilogue is the faster way for a
    prompt portion: "pair" (pairs of CTAs on 256 x 256 tiles), "single" (one CTA on 128 x 256) or None (the
    library's product followed by the gate kernel).  The fused forms save the gate kernel's pass over the
    [rows, 2 I] product.  The pair form runs at the library's rate and wins from 1,024 rows at every width and
    from 512 where the reduction is long; the single-CTA form falls behind the library when the reduction is
    long or the rows are many, and is kept for the short portions of a narrow model
    (measured: profiles/gemm_tc_swiglu__prefill_2048.md)."""
    narrow = weight.shape[1] <= 1536
    if rows >= 1024 or (rows >= 512 and not narrow):
        return "pair"
    return "single" if narrow and rows >= 128 else None


GEMM_TC_GATES = {"silu": 1, "relu": 2}  # the gates that the tcgen05 product's epilogue applies


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
            swiglu_blocks: bool = False, pair: bool = False, activation: str = "silu") -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in TMEM).
    ``swiglu_blocks``: w's rows alternate gate/up in blocks of eight and out is [M, N / 2] = up * act(gate),
    ``activation`` one of ``GEMM_TC_GATES``.
    ``pair``: by pairs of CTAs on 256 x 256 tiles (the paired instruction) instead of single CTAs."""
    _check("gemm_tc.x", x, torch.bfloat16)
    _check("gemm_tc.w", w, torch.bfloat16)
    _check("gemm_tc.out", out)
    M, K = x.shape
    N = w.shape[0]
    want_cols = N // 2 if swiglu_blocks else N
    if w.shape[1] != K or tuple(out.shape) != (M, want_cols) or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"gemm_tc: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} {out.dtype}")
    entry = library().q3_gemm_tc_pair if pair else library().q3_gemm_tc
    code = entry(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, want_cols,
                 1 if out.dtype == torch.float32 else 0, GEMM_TC_GATES[activation] if swiglu_blocks else 0,
                 status.data_ptr(), _stream())
    _done("gemm_tc", code, f"M {M} N {N} K {K}{' pair' if pair else ''}")


# ------------------------------------------------------------------ fast bfloat16 attention
MAX_DECODE_SPLITS = 32


def gemm_tc_qkv_takes(rows: int, x: torch.Tensor, weight: torch.Tensor, head_dim: int, rotary_dim: int) -> bool:
    """Whether the QKV projection with head norm, rotation and cache write in its epilogue takes this
    case: a prompt portion (128 rows or more) in bfloat16, heads of 64 or 128, rotated whole or not at all."""
    return (rows >= 128 and gemm_tc_takes(x, weight) and head_dim in (64, 128) and rotary_dim in (0, head_dim))


def gemm_tc_qkv_pays(rows: int, weight: torch.Tensor) -> Optional[str]:
    """Which projection with ``qkv_post`` as its epilogue is the faster way for a prompt portion: "pair"
    (pairs of CTAs on tiles of 256 rows), "single" (one CTA per tile) or None (the library's product, then
    ``qkv_post``).  The fused forms save ``qkv_post``'s pass over the projection and a launch.  Inside the
    step they win from 256 rows at a reduction up to 1,536 (3 to 6 % of the step); where the reduction is
    longer the step showed no gain over the library's product beyond its spread from run to run
    (profiles/gemm_tc_qkv__prefill_2048.md, profiles/gemm_tc_pair__products.md)."""
    if weight.shape[1] > 1536 or rows < 256:
        return None
    return "pair" if rows >= 1024 else "single"


def gemm_tc_qkv(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                cos_sin: Optional[torch.Tensor], positions: torch.Tensor, tok_seq: torch.Tensor,
                block_table: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, write_kv: bool,
                status: torch.Tensor, pair: bool = False) -> None:
    """x[T, K] @ w[(Hq + 2 Hkv) D, K]^T on the tensor cores with ``qkv_post`` as the epilogue: the
    projection is rounded to bfloat16, normed and rotated head by head and written to ``q_out`` and the
    cache pages; it is never stored itself (``gemm_tc_qkv_pays`` says where the attention part takes it).
    ``pair``: by pairs of CTAs on tiles of 256 rows (the paired instruction) instead of single CTAs."""
    for name, t in (("x", x), ("w", w), ("q_out", q_out), ("k_pages", k_pages), ("v_pages", v_pages)):
        _check(f"gemm_tc_qkv.{name}", t, torch.bfloat16)
    for name, t in (("positions", positions), ("tok_seq", tok_seq), ("block_table", block_table)):
        _check(f"gemm_tc_qkv.{name}", t, torch.int32)
    T, K = x.shape
    width = (num_q_heads + 2 * num_kv_heads) * head_dim
    num_pages, hkv, page_size, d = k_pages.shape
    if (tuple(w.shape) != (width, K) or q_out.numel() != T * num_q_heads * head_dim or hkv != num_kv_heads
            or d != head_dim or v_pages.shape != k_pages.shape or positions.numel() != T or tok_seq.numel() != T
            or block_table.dim() != 2):
        raise KernelError(f"gemm_tc_qkv: x {tuple(x.shape)}, w {tuple(w.shape)}, q_out {tuple(q_out.shape)}, "
                          f"pages {tuple(k_pages.shape)}, heads {num_q_heads}/{num_kv_heads} x {head_dim}")
    for name, wt in (("q_weight", q_weight), ("k_weight", k_weight)):
        if wt is not None:
            _check(f"gemm_tc_qkv.{name}", wt, torch.float32)
            if wt.numel() != head_dim:
                raise KernelError(f"gemm_tc_qkv: {name} has {wt.numel()} elements, head_dim is {head_dim}")
    if cos_sin is not None:
        _check("gemm_tc_qkv.cos_sin", cos_sin, torch.float32)
        if tuple(cos_sin.shape) != (T, head_dim):
            raise KernelError(f"gemm_tc_qkv: cos_sin {tuple(cos_sin.shape)} expected [{T}, {head_dim}]")
    code = library().q3_gemm_tc_qkv(
        x.data_ptr(), w.data_ptr(), T, K, num_q_heads, num_kv_heads, head_dim, _ptr(q_weight), _ptr(k_weight),
        float(eps), _ptr(cos_sin), positions.data_ptr(), tok_seq.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], page_size, k_pages.data_ptr(), v_pages.data_ptr(), num_pages, q_out.data_ptr(),
        1 if write_kv else 0, 1 if pair else 0, status.data_ptr(), _stream())
    _done("gemm_tc_qkv", code, f"T {T} K {K} heads {num_q_heads}/{num_kv_heads} x {head_dim}{' pair' if pair else ''}")


def fast_attention_takes(dtype: torch.dtype, num_q_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core kernels take this shape (else the plain kernel runs)."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and num_q_heads % num_kv_heads == 0 and num_q_heads // num_kv_heads <= 16)


_DEVICE_FACTS = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once)."""
    key = ("sms", torch.cuda.current_device())
    if key not in _DEVICE_FACTS:
        _DEVICE_FACTS[key] = max(1, int(library()._lib.q3_sm_count()))
    return _DEVICE_FACTS[key]


def decode_blocks_per_sm(head_dim: int) -> int:
    """Blocks of the cp.async decode kernel that one SM holds at once, as the CUDA runtime reckons it from the
    compiled kernel (registers, shared memory); asked once per head size."""
    key = ("decode blocks", torch.cuda.current_device(), head_dim)
    if key not in _DEVICE_FACTS:
        _DEVICE_FACTS[key] = max(1, int(library()._lib.q3_attn_decode_blocks_per_sm(int(head_dim))))
    return _DEVICE_FACTS[key]


def decode_tma_takes(head_dim: int, page_size: int) -> bool:
    """Whether the decode kernel with the TMA loader takes this shape (else the cp.async one runs)."""
    return head_dim in (64, 128) and page_size % 16 == 0


def decode_takes_raw_qkv(dtype: torch.dtype, num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                         num_tokens: int, num_seqs: int, num_decode: int) -> bool:
    """Whether the decode attention kernel can do the work of ``qkv_post`` itself: every row of the step
    brings one token and the kernel with the TMA loader takes the shape."""
    return (num_tokens == num_seqs == num_decode and num_decode > 0
            and fast_attention_takes(dtype, num_q_heads, num_kv_heads, head_dim)
            and decode_tma_takes(head_dim, page_size))


DECODE_SATURATING = 2.3    # blocks per SM that together take tiles as fast as the memory gives them
DECODE_LATER_WAVE = 5      # what every wave of blocks after the first costs beside its tiles, in tiles
DECODE_WIDE_GRID = 20      # what the form of the kernel for more blocks per SM costs beside its tiles
DECODE_LONG_BLOCK = (0.15, 128)  # a single wave of that form: per tile of a block beyond so many


def decode_splits(num_seqs: int, num_kv_heads: int, max_kv_len: int, window: int, head_dim: int = 128,
                  blocks_per_sm: Optional[int] = None, wide_blocks_per_sm: Optional[int] = None) -> int:
    """How many ranges a sequence's keys are cut into.  Blocks run in waves of (SMs x blocks per SM).  A
    block alone walks its 16-key tiles at its own pace; ``DECODE_SATURATING`` blocks per SM together take
    tiles as fast as the memory gives them, and more blocks then only share that rate; every wave after the
    first costs a start.  So a wave of n blocks of L tiles costs max(L, n L / saturating), and the count with
    the least sum over its waves wins, the smaller count on a tie.  ``wide_blocks_per_sm``: the kernel has a
    form with that many (smaller) blocks per SM, which the launcher takes for a grid that ``blocks_per_sm``
    do not hold at once.  The constants are fitted to sweeps of the decode step over batch and context
    (profiles/attn_decode_tma__decode_b8_ctx4096.md)."""
    span = min(max_kv_len, window) if window and window > 0 else max_kv_len
    tiles = max(1, -(-span // 16))
    sms = sm_count()
    narrow = sms * (blocks_per_sm or decode_blocks_per_sm(head_dim))
    saturating = DECODE_SATURATING * sms
    pairs = max(1, num_seqs * num_kv_heads)
    best, best_cost = 1, None
    for s in range(1, MAX_DECODE_SPLITS + 1):
        if s > 1 and tiles // s < 4:
            break
        per_block = -(-tiles // s)
        blocks = pairs * s
        wide = wide_blocks_per_sm is not None and blocks > narrow
        slots = sms * wide_blocks_per_sm if wide else narrow
        full, rest = divmod(blocks, slots)
        waves = full + (1 if rest else 0)
        cost = full * max(per_block, slots * per_block / saturating) + DECODE_LATER_WAVE * (waves - 1)
        if rest:
            cost += max(per_block, rest * per_block / saturating)
        if wide:
            cost += DECODE_WIDE_GRID
            if waves == 1:
                cost += DECODE_LONG_BLOCK[0] * max(0, per_block - DECODE_LONG_BLOCK[1])
        if best_cost is None or cost < best_cost - 1e-6:
            best, best_cost = s, cost
    return best


def decode_partial_numel(num_seqs: int, num_q_heads: int, head_dim: int) -> int:
    return num_seqs * num_q_heads * MAX_DECODE_SPLITS * (head_dim + 2)


def _attn_common(name, q, k_pages, v_pages, out, q_start, kv_len, block_table):
    _check(f"{name}.q", q, torch.bfloat16)
    _check(f"{name}.out", out, torch.bfloat16)
    _check(f"{name}.k_pages", k_pages, torch.bfloat16)
    _check(f"{name}.v_pages", v_pages, torch.bfloat16)
    for nm, t in (("q_start", q_start), ("kv_len", kv_len), ("block_table", block_table)):
        _check(f"{name}.{nm}", t, torch.int32)
    T, Hq, D = q.shape
    num_pages, Hkv, page_size, d = k_pages.shape
    if d != D or v_pages.shape != k_pages.shape or out.numel() != q.numel() or block_table.dim() != 2:
        raise KernelError(f"{name}: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    return T, Hq, D, num_pages, Hkv, page_size


def attn_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                partial: Optional[torch.Tensor], q_start: torch.Tensor, kv_len: torch.Tensor,
                block_table: torch.Tensor, num_seqs: int, scale: float, window: int, num_splits: int,
                status: torch.Tensor, loader: str = "cp_async", raw_qkv=None) -> None:
    """Split-KV tensor-core attention for the first ``num_seqs`` rows, one query token each.
    ``raw_qkv = (qkv, q_weight, k_weight, eps, cos_sin, write_kv)`` (TMA loader only): ``q`` only gives the
    shape; the kernel norms and rotates the query from the raw projection ``qkv[T, (Hq + 2 Hkv) D]`` itself
    and makes, stores and uses the new key and value (the work of ``qkv_post`` for these tokens).
    ``loader``: ``"cp_async"`` (every warp copies its own tiles) or ``"tma"`` (a loader warp feeds a
    ring of stages through TMA; head size 64 / 128 and pages that are multiples of 16 only)."""
    T, Hq, D, num_pages, Hkv, page_size = _attn_common("attn_decode", q, k_pages, v_pages, out, q_start, kv_len,
                                                        block_table)
    if num_seqs > kv_len.numel() or num_seqs > block_table.shape[0]:
        raise KernelError(f"attn_decode: {num_seqs} sequences, {kv_len.numel()} lengths")
    if num_splits > 1:
        if partial is None:
            raise KernelError("attn_decode: more than one split needs scratch memory")
        _check("attn_decode.partial", partial, torch.float32)
        if partial.numel() < num_seqs * Hq * num_splits * (D + 2):
            raise KernelError(f"attn_decode: scratch of {partial.numel()} floats is too small for {num_seqs} "
                              f"sequences x {Hq} heads x {num_splits} splits")
    if raw_qkv is not None:
        qkv, q_weight, k_weight, eps, cos_sin, write_kv = raw_qkv
        if loader != "tma":
            raise KernelError("attn_decode: only the kernel with the TMA loader takes the raw projection")
        _check("attn_decode.qkv", qkv, torch.bfloat16)
        if tuple(qkv.shape) != (T, (Hq + 2 * Hkv) * D) or num_seqs > T:
            raise KernelError(f"attn_decode: raw projection {tuple(qkv.shape)} for {T} tokens of {Hq}+2x{Hkv} heads of {D}")
        for nm, t, n in (("q_weight", q_weight, D), ("k_weight", k_weight, D), ("cos_sin", cos_sin, T * D)):
            if t is not None:
                _check(f"attn_decode.{nm}", t, torch.float32)
                if t.numel() != n:
                    raise KernelError(f"attn_decode: {nm} has {t.numel()} values, {n} expected")
        code = library().q3_attn_decode_tma_qkv(
            qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos_sin), 1 if write_kv else 0,
            k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), _ptr(partial), q_start.data_ptr(), kv_len.data_ptr(),
            block_table.data_ptr(), block_table.shape[1], page_size, num_pages, num_seqs, Hq, Hkv, D, float(scale),
            int(window), int(num_splits), status.data_ptr(), _stream())
        _done("attn_decode", code, f"heads {Hq}/{Hkv}, head_dim {D}, page {page_size}, raw projection")
        return
    fn = library().q3_attn_decode_tma if loader == "tma" else library().q3_attn_decode
    code = fn(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
              _ptr(partial), q_start.data_ptr(), kv_len.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], page_size, num_pages, num_seqs, Hq, Hkv, D, float(scale),
              int(window), int(num_splits), status.data_ptr(), _stream())
    _done("attn_decode", code, f"heads {Hq}/{Hkv}, head_dim {D}, page {page_size}, loader {loader}")


def attn_prefill(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                 q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor, num_seqs: int,
                 max_q_len: int, scale: float, window: int, status: torch.Tensor) -> None:
    """Tensor-core attention for ``num_seqs`` rows of any query length (q_start has num_seqs + 1 entries)."""
    T, Hq, D, num_pages, Hkv, page_size = _attn_common("attn_prefill", q, k_pages, v_pages, out, q_start, kv_len,
                                                        block_table)
    if q_start.numel() < num_seqs + 1 or kv_len.numel() < num_seqs or block_table.shape[0] < num_seqs:
        raise KernelError(f"attn_prefill: {num_seqs} sequences, q_start {q_start.numel()}, kv_len {kv_len.numel()}")
    code = library().q3_attn_prefill(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                                     q_start.data_ptr(), kv_len.data_ptr(), block_table.data_ptr(),
                                     block_table.shape[1], page_size, num_pages, num_seqs, int(max_q_len), Hq, Hkv, D,
                                     float(scale), int(window), status.data_ptr(), _stream())
    _done("attn_prefill", code, f"heads {Hq}/{Hkv}, head_dim {D}")


def attn_tc_takes(head_dim: int, page_size: int, window: int) -> bool:
    """Whether the tcgen05 portion kernel takes this shape (else the mma.sync one runs)."""
    return head_dim in (64, 128) and page_size in (8, 16, 32, 64) and not (window and window > 0)


def attn_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
            q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor, num_seqs: int,
            max_q_len: int, scale: float, status: torch.Tensor) -> None:
    """Portion attention on the tcgen05 tensor cores: TMA-fed pages, S and O in tensor memory."""
    T, Hq, D, num_pages, Hkv, page_size = _attn_common("attn_tc", q, k_pages, v_pages, out, q_start, kv_len,
                                                        block_table)
    if q_start.numel() < num_seqs + 1 or kv_len.numel() < num_seqs or block_table.shape[0] < num_seqs:
        raise KernelError(f"attn_tc: {num_seqs} sequences, q_start {q_start.numel()}, kv_len {kv_len.numel()}")
    code = library().q3_attn_tc(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                                q_start.data_ptr(), kv_len.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                page_size, num_pages, num_seqs, int(max_q_len), Hq, Hkv, D, float(scale),
                                status.data_ptr(), _stream())
    _done("attn_tc", code, f"heads {Hq}/{Hkv}, head_dim {D}, page {page_size}")


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                    q_start: torch.Tensor, kv_len: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
                    num_seqs: int, num_decode: int, max_q_len: int, max_kv_len: int, scale: float, window: int,
                    status: torch.Tensor, partial: Optional[torch.Tensor] = None,
                    portion_kernel: str = "auto", decode_kernel: str = "auto", raw_qkv=None) -> None:
    """``raw_qkv``: see ``attn_decode``; only where ``decode_takes_raw_qkv`` says so.
    Causal attention of a mixed batch over the pages: rows [0, num_decode) bring one token each and
    go to the split-KV decode kernel, the rest to a portion kernel (tcgen05 where it takes the shape,
    else mma.sync; ``portion_kernel="mma"`` forces the latter); shapes no tensor-core kernel takes
    (and float32) go to the plain kernel."""
    T, Hq, D = q.shape
    Hkv = k_pages.shape[1]
    if block_table.dim() != 2 or max_kv_len > block_table.shape[1] * k_pages.shape[2]:
        raise KernelError(f"paged_attention: the longest request has {max_kv_len} tokens, a block table row of "
                          f"{block_table.shape[-1]} pages of {k_pages.shape[2]} holds fewer")
    if not fast_attention_takes(q.dtype, Hq, Hkv, D):
        attn_ref(q, k_pages, v_pages, out, q_start, kv_len, tok_seq, block_table, scale, window, status)
        return
    if num_decode > 0:
        tma = decode_kernel != "cp_async" and decode_tma_takes(D, k_pages.shape[2])
        if tma:
            # The kernel is compiled for two, three and four blocks per SM (the last with fewer warps and
            # stages per block) and takes the smallest form that holds the grid at once, the last for all larger grids.
            splits = decode_splits(num_decode, Hkv, max_kv_len, window, D, blocks_per_sm=3, wide_blocks_per_sm=4)
        else:
            splits = decode_splits(num_decode, Hkv, max_kv_len, window, D)
        if partial is None or partial.numel() < num_decode * Hq * splits * (D + 2):
            splits = 1 if partial is None else max(1, partial.numel() // (num_decode * Hq * (D + 2)))
        attn_decode(q, k_pages, v_pages, out, partial, q_start, kv_len, block_table, num_decode, scale, window,
                    splits, status, loader="tma" if tma else "cp_async", raw_qkv=raw_qkv)
    elif raw_qkv is not None:
        raise KernelError("paged_attention: the raw projection is only taken by a step of single tokens")
    if num_seqs > num_decode:
        rest = (q_start[num_decode:], kv_len[num_decode:], block_table[num_decode:], num_seqs - num_decode, max_q_len)
        if portion_kernel != "mma" and attn_tc_takes(D, k_pages.shape[2], window):
            attn_tc(q, k_pages, v_pages, out, *rest, scale, status)
        else:
            attn_prefill(q, k_pages, v_pages, out, *rest, scale, window, status)


# ------------------------------------------------------------------ state carried from token to token
def token_shift(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, tok_seq: torch.Tensor,
                slot_ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[t] = x[t] + (x[t - 1] - x[t]) * mu, the token before a portion's first one taken from ``state``
    (float32 [slots, W], zero for a new request), which then receives the portion's last x."""
    _check("token_shift.x", x, torch.float32)
    _check("token_shift.mu", mu, torch.float32)
    _check("token_shift.state", state, torch.float32)
    _check("token_shift.out", out)
    for name, t in (("q_start", q_start), ("tok_seq", tok_seq), ("slot_ids", slot_ids)):
        _check(f"token_shift.{name}", t, torch.int32)
    T, W = x.shape
    if tuple(out.shape) != (T, W) or mu.numel() != W or state.dim() != 2 or state.shape[1] != W or tok_seq.numel() != T:
        raise KernelError(f"token_shift: x {tuple(x.shape)}, out {tuple(out.shape)}, mu {tuple(mu.shape)}, "
                          f"state {tuple(state.shape)}")
    code = library().q3_token_shift(x.data_ptr(), mu.data_ptr(), state.data_ptr(), q_start.data_ptr(), tok_seq.data_ptr(),
                                    slot_ids.data_ptr(), out.data_ptr(), dtype_tag(out.dtype), T, W, state.shape[0],
                                    status.data_ptr(), _stream())
    _done("token_shift", code)


def causal_conv(x: torch.Tensor, column: int, in_bias: Optional[torch.Tensor], weight: torch.Tensor,
                bias: Optional[torch.Tensor], state: torch.Tensor, q_start: torch.Tensor, tok_seq: torch.Tensor,
                slot_ids: torch.Tensor, num_seqs: int, out: torch.Tensor, activation: str, status: torch.Tensor) -> None:
    """A short causal convolution per channel over the columns ``column .. column + C`` of ``x`` [T, ld]:
    out[t, c] = act(sum_j weight[c, j] * v[t - (K - 1 - j), c] + bias[c]), v = x + in_bias; what lies before a
    portion comes from ``state`` (float32 [slots, K - 1, C], zero for a new request), which is renewed."""
    _check("causal_conv.x", x)
    _check("causal_conv.out", out, x.dtype)
    _check("causal_conv.weight", weight, torch.float32)
    _check("causal_conv.state", state, torch.float32)
    for name, t in (("q_start", q_start), ("tok_seq", tok_seq), ("slot_ids", slot_ids)):
        _check(f"causal_conv.{name}", t, torch.int32)
    T, ld = x.shape
    C, K = weight.shape
    if (tuple(out.shape) != (T, C) or column < 0 or column + C > ld or state.dim() != 3
            or tuple(state.shape[1:]) != (K - 1, C) or tok_seq.numel() != T or q_start.numel() < num_seqs + 1):
        raise KernelError(f"causal_conv: x {tuple(x.shape)} column {column}, weight {tuple(weight.shape)}, out "
                          f"{tuple(out.shape)}, state {tuple(state.shape)}")
    for name, t in (("in_bias", in_bias), ("bias", bias)):
        if t is not None:
            _check(f"causal_conv.{name}", t, torch.float32)
            if t.numel() != C:
                raise KernelError(f"causal_conv: {name} has {t.numel()} values for {C} channels")
    code = library().q3_causal_conv(x.data_ptr() + column * x.element_size(), ld, _ptr(in_bias), weight.data_ptr(),
                                    _ptr(bias), state.data_ptr(), q_start.data_ptr(), tok_seq.data_ptr(),
                                    slot_ids.data_ptr(), out.data_ptr(), dtype_tag(x.dtype), T, int(num_seqs), C, K,
                                    activation_code(activation), state.shape[0], status.data_ptr(), _stream())
    _done("causal_conv", code, f"channels {C}, taps {K}")


BLOCK_DIAG_FEW_ROWS = 16  # up to so many tokens the engine's own kernel streams the weight once


def block_diag(u: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[b, t, r] = sum_e weight[b, r, e] * u[t, b * bw + e]: a block-diagonal product, float32 result
    [blocks, T, rows].  u [T, blocks * bw] and weight [blocks, rows, bw] in one dtype.  bfloat16 with more than
    ``BLOCK_DIAG_FEW_ROWS`` tokens: the library's batched product; otherwise the engine's own kernel."""
    _check("block_diag.u", u)
    _check("block_diag.weight", weight, u.dtype)
    _check("block_diag.out", out, torch.float32)
    T, C = u.shape
    nb, rows, bw = weight.shape
    if nb * bw != C or tuple(out.shape) != (nb, T, rows):
        raise KernelError(f"block_diag: u {tuple(u.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if u.dtype == torch.bfloat16 and T > BLOCK_DIAG_FEW_ROWS:
        torch.bmm(u.view(T, nb, bw).transpose(0, 1), weight.transpose(1, 2), out_dtype=torch.float32, out=out)
        return
    code = library().q3_block_diag(u.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_tag(u.dtype), T, nb, bw, rows,
                                   _stream())
    _done("block_diag", code, f"blocks {nb} of {bw}")


def scan_chunk() -> int:
    """Tokens per chunk of the chunked scans."""
    if "scan chunk" not in _DEVICE_FACTS:
        _DEVICE_FACTS["scan chunk"] = int(library()._lib.q3_scan_chunk())
    return _DEVICE_FACTS["scan chunk"]


def scan_chunk_records(num_tokens: int, num_seqs: int) -> int:
    """Chunk records that the chunked scans' scratch must hold for a step of so many tokens and requests."""
    return num_tokens // scan_chunk() + num_seqs + 1


def scan_chunked_pays(dtype: torch.dtype, max_q_len: int) -> bool:
    """Whether a step's recurrences run over chunks of their portions: bfloat16 runs with a portion of at least
    four chunks.  A thread per channel that walks a whole portion keeps few SMs busy; the float32 run keeps that
    walk all the same, so that its bits do not depend on how a prompt was cut."""
    return dtype == torch.bfloat16 and max_q_len >= 4 * scan_chunk()


def rglru_scan(proj: torch.Tensor, y_column: int, y_bias: Optional[torch.Tensor], u: torch.Tensor, gates: torch.Tensor,
               ra_bias: torch.Tensor, ri_bias: torch.Tensor, lam: torch.Tensor, decay: float, state: torch.Tensor,
               q_start: torch.Tensor, slot_ids: torch.Tensor, num_seqs: int, out: torch.Tensor,
               status: torch.Tensor, max_q_len: int = 0, scratch: Optional[torch.Tensor] = None) -> None:
    """The gated linear recurrence S = a S + sqrt(1 - a^2) (i * u) with a = exp(-decay * softplus(lam) * r),
    r and i the sigmoids of ``gates`` (float32 [blocks, T, 2 bw]: per block the recurrence gate's rows, then the
    input gate's) plus their biases; out = S * gelu_tanh(proj[:, y_column : y_column + C] + y_bias).  ``state``:
    float32 [slots, C].  With ``scratch`` (float32, ``scan_chunk_records(T, num_seqs) * 2 * C``) and a longest
    portion ``max_q_len`` of ``scan_chunked_pays`` the portions are cut into chunks that run side by side."""
    _check("rglru_scan.proj", proj)
    _check("rglru_scan.u", u, proj.dtype)
    _check("rglru_scan.out", out, proj.dtype)
    _check("rglru_scan.gates", gates, torch.float32)
    _check("rglru_scan.state", state, torch.float32)
    T, C = u.shape
    nb, Tg, two_bw = gates.shape
    for name, t in (("ra_bias", ra_bias), ("ri_bias", ri_bias), ("lam", lam)) + ((("y_bias", y_bias),) if y_bias is not None else ()):
        _check(f"rglru_scan.{name}", t, torch.float32)
        if t.numel() != C:
            raise KernelError(f"rglru_scan: {name} has {t.numel()} values for {C} channels")
    if (Tg != T or nb * two_bw != 2 * C or tuple(out.shape) != (T, C) or proj.shape[0] != T or y_column < 0
            or y_column + C > proj.shape[1] or state.dim() != 2 or state.shape[1] != C):
        raise KernelError(f"rglru_scan: proj {tuple(proj.shape)}, u {tuple(u.shape)}, gates {tuple(gates.shape)}, "
                          f"state {tuple(state.shape)}")
    if scratch is not None and scan_chunked_pays(proj.dtype, max_q_len):
        _check("rglru_scan.scratch", scratch, torch.float32)
        if scratch.numel() < scan_chunk_records(T, num_seqs) * 2 * C:
            raise KernelError(f"rglru_scan: scratch of {scratch.numel()} floats for {T} tokens of {num_seqs} requests")
        code = library().q3_rglru_scan_chunked(
            proj.data_ptr(), proj.shape[1], int(y_column), _ptr(y_bias), u.data_ptr(), gates.data_ptr(),
            ra_bias.data_ptr(), ri_bias.data_ptr(), lam.data_ptr(), float(decay), state.data_ptr(), scratch.data_ptr(),
            q_start.data_ptr(), slot_ids.data_ptr(), out.data_ptr(), dtype_tag(proj.dtype), T, int(num_seqs),
            int(max_q_len), C, two_bw // 2, state.shape[0], status.data_ptr(), _stream())
        _done("rglru_scan (chunked)", code, f"channels {C}")
        return
    code = library().q3_rglru_scan(proj.data_ptr(), proj.shape[1], int(y_column), _ptr(y_bias), u.data_ptr(),
                                   gates.data_ptr(), ra_bias.data_ptr(), ri_bias.data_ptr(), lam.data_ptr(), float(decay),
                                   state.data_ptr(), q_start.data_ptr(), slot_ids.data_ptr(), out.data_ptr(),
                                   dtype_tag(proj.dtype), T, int(num_seqs), C, two_bw // 2, state.shape[0],
                                   status.data_ptr(), _stream())
    _done("rglru_scan", code, f"channels {C}")


def selective_scan(xc: torch.Tensor, proj: torch.Tensor, z_column: int, bc: torch.Tensor, dt: torch.Tensor,
                   dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor,
                   q_start: torch.Tensor, slot_ids: torch.Tensor, num_seqs: int, out: torch.Tensor,
                   status: torch.Tensor, max_q_len: int = 0, scratch: Optional[torch.Tensor] = None) -> None:
    """The selective scan: per channel c and state n, S = exp(step A[c, n]) S + step x B[n], y = sum_n S C[n] +
    D x, out = y * silu(z); step = softplus(dt + dt_bias), A = -exp(a_log), z = proj[:, z_column : z_column + I];
    bc: float32 [T, 2 N] (B then C); dt: float32 [T, I]; state: float32 [slots, N, I].  ``scratch`` (float32,
    ``scan_chunk_records(T, num_seqs) * (N + 1) * I``) and ``max_q_len``: as in ``rglru_scan``."""
    _check("selective_scan.xc", xc)
    _check("selective_scan.proj", proj, xc.dtype)
    _check("selective_scan.out", out, xc.dtype)
    for name, t in (("bc", bc), ("dt", dt), ("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip), ("state", state)):
        _check(f"selective_scan.{name}", t, torch.float32)
    T, I = xc.shape
    N = a_log.shape[1]
    if (tuple(a_log.shape) != (I, N) or tuple(bc.shape) != (T, 2 * N) or tuple(dt.shape) != (T, I) or dt_bias.numel() != I
            or d_skip.numel() != I or tuple(out.shape) != (T, I) or proj.shape[0] != T or z_column < 0
            or z_column + I > proj.shape[1] or state.dim() != 3 or tuple(state.shape[1:]) != (N, I)):
        raise KernelError(f"selective_scan: x {tuple(xc.shape)}, proj {tuple(proj.shape)}, bc {tuple(bc.shape)}, dt "
                          f"{tuple(dt.shape)}, A {tuple(a_log.shape)}, state {tuple(state.shape)}")
    if scratch is not None and scan_chunked_pays(xc.dtype, max_q_len):
        _check("selective_scan.scratch", scratch, torch.float32)
        if scratch.numel() < scan_chunk_records(T, num_seqs) * (N + 1) * I:
            raise KernelError(f"selective_scan: scratch of {scratch.numel()} floats for {T} tokens of {num_seqs} requests")
        code = library().q3_selective_scan_chunked(
            xc.data_ptr(), proj.data_ptr(), proj.shape[1], int(z_column), bc.data_ptr(), dt.data_ptr(), dt_bias.data_ptr(),
            a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), scratch.data_ptr(), q_start.data_ptr(),
            slot_ids.data_ptr(), out.data_ptr(), dtype_tag(xc.dtype), T, int(num_seqs), int(max_q_len), I, N,
            state.shape[0], status.data_ptr(), _stream())
        _done("selective_scan (chunked)", code, f"channels {I}, state {N}")
        return
    code = library().q3_selective_scan(xc.data_ptr(), proj.data_ptr(), proj.shape[1], int(z_column), bc.data_ptr(),
                                       dt.data_ptr(), dt_bias.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(),
                                       state.data_ptr(), q_start.data_ptr(), slot_ids.data_ptr(), out.data_ptr(),
                                       dtype_tag(xc.dtype), T, int(num_seqs), I, N, state.shape[0], status.data_ptr(),
                                       _stream())
    _done("selective_scan", code, f"channels {I}, state {N}")


# ------------------------------------------------------------------ attention without a softmax
def qk_gate_post(proj: torch.Tensor, q_out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                 q_weight: torch.Tensor, k_weight: torch.Tensor, eps: float, temp_coef: float, temp_every: int,
                 positions: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor, num_q_heads: int,
                 num_kv_heads: int, head_dim: int, gate_out: Optional[torch.Tensor], write_kv: bool,
                 status: torch.Tensor) -> None:
    """From a step's projection [T, (Hq + Hkv) D (+ Hq)]: q normed per head, times the temperature
    1 + coef * ln(floor((p + 1) / every) + 1) (``temp_every`` <= 0: none), to ``q_out``; k normed per head into
    plane k of the pages and as projected into plane v; sigmoid of the last Hq columns to ``gate_out``."""
    _check("qk_gate_post.proj", proj)
    for name, t in (("q_out", q_out), ("k_pages", k_pages), ("v_pages", v_pages)):
        _check(f"qk_gate_post.{name}", t, proj.dtype)
    for name, t in (("positions", positions), ("tok_seq", tok_seq), ("block_table", block_table)):
        _check(f"qk_gate_post.{name}", t, torch.int32)
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight)):
        _check(f"qk_gate_post.{name}", t, torch.float32)
        if t.numel() != head_dim:
            raise KernelError(f"qk_gate_post: {name} has {t.numel()} values, the heads are {head_dim} wide")
    T, ld = proj.shape
    need = (num_q_heads + num_kv_heads) * head_dim + (num_q_heads if gate_out is not None else 0)
    num_pages, hkv, page_size, d = k_pages.shape
    if (ld != need or q_out.numel() != T * num_q_heads * head_dim or hkv != num_kv_heads or d != head_dim
            or v_pages.shape != k_pages.shape or positions.numel() != T or tok_seq.numel() != T or block_table.dim() != 2):
        raise KernelError(f"qk_gate_post: proj {tuple(proj.shape)} expected [T, {need}], q_out {tuple(q_out.shape)}, "
                          f"pages {tuple(k_pages.shape)}")
    if gate_out is not None:
        _check("qk_gate_post.gate_out", gate_out, torch.float32)
        if gate_out.numel() != T * num_q_heads:
            raise KernelError(f"qk_gate_post: gate_out {tuple(gate_out.shape)} for {T} tokens of {num_q_heads} heads")
    code = library().q3_qk_gate_post(proj.data_ptr(), dtype_tag(proj.dtype), T, ld, num_q_heads, num_kv_heads, head_dim,
                                     q_weight.data_ptr(), k_weight.data_ptr(), float(eps), float(temp_coef),
                                     int(temp_every), positions.data_ptr(), tok_seq.data_ptr(), block_table.data_ptr(),
                                     block_table.shape[1], page_size, k_pages.data_ptr(), v_pages.data_ptr(), num_pages,
                                     q_out.data_ptr(), _ptr(gate_out), 1 if write_kv else 0, status.data_ptr(), _stream())
    _done("qk_gate_post", code, f"heads {num_q_heads}/{num_kv_heads} x {head_dim}")


def attn_sigmoid(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                 head_bias: Optional[torch.Tensor], gate: Optional[torch.Tensor], q_start: torch.Tensor,
                 kv_len: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor, scale: float,
                 status: torch.Tensor) -> None:
    """Plain paged causal attention with sigmoid weights (one warp per query and head), any head size up to
    512: out = gate * sum_n sigmoid(q . k_n * scale + head_bias[h]) v_n."""
    _check("attn_sigmoid.q", q)
    _check("attn_sigmoid.out", out, q.dtype)
    _check("attn_sigmoid.k_pages", k_pages, q.dtype)
    _check("attn_sigmoid.v_pages", v_pages, q.dtype)
    for name, t in (("q_start", q_start), ("kv_len", kv_len), ("tok_seq", tok_seq), ("block_table", block_table)):
        _check(f"attn_sigmoid.{name}", t, torch.int32)
    T, Hq, D = q.shape
    num_pages, Hkv, page_size, d = k_pages.shape
    if d != D or v_pages.shape != k_pages.shape or out.numel() != q.numel() or block_table.dim() != 2:
        raise KernelError(f"attn_sigmoid: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    for name, t, n in (("head_bias", head_bias, Hq), ("gate", gate, T * Hq)):
        if t is not None:
            _check(f"attn_sigmoid.{name}", t, torch.float32)
            if t.numel() != n:
                raise KernelError(f"attn_sigmoid: {name} has {t.numel()} values, {n} expected")
    code = library().q3_attn_sigmoid(q.data_ptr(), dtype_tag(q.dtype), k_pages.data_ptr(), v_pages.data_ptr(),
                                     out.data_ptr(), _ptr(head_bias), _ptr(gate), q_start.data_ptr(), kv_len.data_ptr(),
                                     tok_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
                                     num_pages, T, Hq, Hkv, D, float(scale), status.data_ptr(), _stream())
    _done("attn_sigmoid", code, f"heads {Hq}/{Hkv}, head_dim {D}")


SIGMOID_MAX_SPLITS = 32


def sigmoid_attention_fast(dtype: torch.dtype, num_q_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core kernel takes the shape (else the plain one runs)."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256 and num_q_heads % num_kv_heads == 0


def sigmoid_partial_numel(num_seqs: int, num_q_heads: int, head_dim: int) -> int:
    return num_seqs * SIGMOID_MAX_SPLITS * num_q_heads * head_dim


def sigmoid_decode_splits(num_seqs: int, num_kv_heads: int, max_kv_len: int) -> int:
    """Key ranges per sequence of the decode form: enough blocks for two per SM, but no range under four
    tiles of 64 keys."""
    tiles = max(1, -(-max_kv_len // 64))
    want = -(-2 * sm_count() // max(1, num_seqs * num_kv_heads))
    return max(1, min(SIGMOID_MAX_SPLITS, tiles // 4, want))


def attn_sigmoid_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                     head_bias: Optional[torch.Tensor], gate: Optional[torch.Tensor], q_start: torch.Tensor,
                     kv_len: torch.Tensor, block_table: torch.Tensor, num_seqs: int, max_q_len: int, scale: float,
                     status: torch.Tensor, decode: bool = False, num_splits: int = 1,
                     partial: Optional[torch.Tensor] = None) -> None:
    """The tensor-core kernel for ``num_seqs`` rows of the batch (q_start has num_seqs + 1 entries): portions of
    any length, or with ``decode`` one token per row, the keys cut into ``num_splits`` ranges."""
    T, Hq, D, num_pages, Hkv, page_size = _attn_common("attn_sigmoid_mma", q, k_pages, v_pages, out, q_start, kv_len,
                                                        block_table)
    if q_start.numel() < num_seqs + (0 if decode else 1) or kv_len.numel() < num_seqs or block_table.shape[0] < num_seqs:
        raise KernelError(f"attn_sigmoid_mma: {num_seqs} sequences, q_start {q_start.numel()}, kv_len {kv_len.numel()}")
    for name, t, n in (("head_bias", head_bias, Hq), ("gate", gate, T * Hq)):
        if t is not None:
            _check(f"attn_sigmoid_mma.{name}", t, torch.float32)
            if t.numel() != n:
                raise KernelError(f"attn_sigmoid_mma: {name} has {t.numel()} values, {n} expected")
    if decode and num_splits > 1:
        if partial is None:
            raise KernelError("attn_sigmoid_mma: more than one key range needs scratch memory")
        _check("attn_sigmoid_mma.partial", partial, torch.float32)
        if partial.numel() < num_seqs * num_splits * Hq * D:
            raise KernelError(f"attn_sigmoid_mma: scratch of {partial.numel()} floats for {num_seqs} x {num_splits} ranges")
    code = library().q3_attn_sigmoid_mma(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                                         _ptr(partial), _ptr(head_bias), _ptr(gate), q_start.data_ptr(), kv_len.data_ptr(),
                                         block_table.data_ptr(), block_table.shape[1], page_size, num_pages, num_seqs,
                                         int(max_q_len), Hq, Hkv, D, float(scale), 1 if decode else 0, int(num_splits),
                                         status.data_ptr(), _stream())
    _done("attn_sigmoid_mma", code, f"heads {Hq}/{Hkv}, head_dim {D}")


def attn_sigmoid_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                    head_bias: Optional[torch.Tensor], gate: Optional[torch.Tensor], q_start: torch.Tensor,
                    kv_len: torch.Tensor, block_table: torch.Tensor, num_seqs: int, max_q_len: int, scale: float,
                    status: torch.Tensor) -> None:
    """Portions with sigmoid weights on the tcgen05 tensor cores (the kernel of ``attn_tc`` with the softmax
    taken out): head size 64 or 128, pages of 8 to 64 tokens."""
    T, Hq, D, num_pages, Hkv, page_size = _attn_common("attn_sigmoid_tc", q, k_pages, v_pages, out, q_start, kv_len,
                                                        block_table)
    if q_start.numel() < num_seqs + 1 or kv_len.numel() < num_seqs or block_table.shape[0] < num_seqs:
        raise KernelError(f"attn_sigmoid_tc: {num_seqs} sequences, q_start {q_start.numel()}, kv_len {kv_len.numel()}")
    for name, t, n in (("head_bias", head_bias, Hq), ("gate", gate, T * Hq)):
        if t is not None:
            _check(f"attn_sigmoid_tc.{name}", t, torch.float32)
            if t.numel() != n:
                raise KernelError(f"attn_sigmoid_tc: {name} has {t.numel()} values, {n} expected")
    code = library().q3_attn_sigmoid_tc(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                                        _ptr(head_bias), _ptr(gate), q_start.data_ptr(), kv_len.data_ptr(),
                                        block_table.data_ptr(), block_table.shape[1], page_size, num_pages, num_seqs,
                                        int(max_q_len), Hq, Hkv, D, float(scale), status.data_ptr(), _stream())
    _done("attn_sigmoid_tc", code, f"heads {Hq}/{Hkv}, head_dim {D}, page {page_size}")


def sigmoid_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                      head_bias: Optional[torch.Tensor], gate: Optional[torch.Tensor], q_start: torch.Tensor,
                      kv_len: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor, num_seqs: int,
                      num_decode: int, max_q_len: int, max_kv_len: int, scale: float, status: torch.Tensor,
                      partial: Optional[torch.Tensor] = None, kernel: str = "auto") -> None:
    """Causal attention with sigmoid weights of a mixed batch over the pages (see ``attn_sigmoid``): rows
    [0, num_decode) bring one token each and go to the decode form of the tensor-core kernel, the rest to its
    portion form, or for heads of 64 or 128 and pages of 8 to 64 tokens to the tcgen05 kernel (``kernel="mma"``
    keeps them on mma.sync); float32, shapes it refuses and ``kernel="plain"`` go to the plain kernel."""
    T, Hq, D = q.shape
    Hkv = k_pages.shape[1]
    if block_table.dim() != 2 or max_kv_len > block_table.shape[1] * k_pages.shape[2]:
        raise KernelError(f"sigmoid_attention: the longest request has {max_kv_len} tokens, a block table row of "
                          f"{block_table.shape[-1]} pages of {k_pages.shape[2]} holds fewer")
    if kernel == "plain" or not sigmoid_attention_fast(q.dtype, Hq, Hkv, D):
        attn_sigmoid(q, k_pages, v_pages, out, head_bias, gate, q_start, kv_len, tok_seq, block_table, scale, status)
        return
    decode = num_decode if Hq // Hkv <= 16 else 0  # a wider group's single tokens run as portions of one
    if decode > 0:
        splits = sigmoid_decode_splits(decode, Hkv, max_kv_len)
        if partial is None or partial.numel() < decode * splits * Hq * D:
            splits = 1 if partial is None else max(1, partial.numel() // (decode * Hq * D))
        attn_sigmoid_mma(q, k_pages, v_pages, out, head_bias, gate, q_start, kv_len, block_table, decode, 1, scale,
                         status, decode=True, num_splits=splits, partial=partial)
    if num_seqs > decode:
        rest = (q_start[decode:], kv_len[decode:], block_table[decode:], num_seqs - decode, max_q_len, scale, status)
        if kernel != "mma" and max_q_len > 1 and attn_tc_takes(D, k_pages.shape[2], 0):
            attn_sigmoid_tc(q, k_pages, v_pages, out, head_bias, gate, *rest)
        else:
            attn_sigmoid_mma(q, k_pages, v_pages, out, head_bias, gate, *rest)


# ------------------------------------------------------------------ several residual streams
HC_MAX_STREAMS = 8


def embed_scaled(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float, status: torch.Tensor) -> None:
    """out[t, s] = float32(table[ids[t]]) * scale for every stream s; out: float32 [T, S, W]."""
    _check("embed_scaled.table", table)
    _check("embed_scaled.ids", ids, torch.int32)
    _check("embed_scaled.out", out, torch.float32)
    T, S, W = out.shape
    if table.shape[1] != W or ids.numel() != T:
        raise KernelError(f"embed_scaled: table {tuple(table.shape)}, ids {tuple(ids.shape)}, out {tuple(out.shape)}")
    code = library().q3_embed_scaled(table.data_ptr(), dtype_tag(table.dtype), ids.data_ptr(), out.data_ptr(), T, W,
                                     table.shape[0], S, float(scale), status.data_ptr(), _stream())
    _done("embed_scaled", code, f"streams {S}")


def _hc_pending(name: str, pending, T: int, S: int, W: int, dtype: torch.dtype):
    if pending is None:
        return None, None, None
    delta, mix, write = pending
    _check(f"{name}.delta", delta, dtype)
    _check(f"{name}.mix", mix, torch.float32)
    _check(f"{name}.write", write, torch.float32)
    if tuple(delta.shape) != (T, W) or tuple(mix.shape) != (S, S) or write.numel() != S:
        raise KernelError(f"{name}: delta {tuple(delta.shape)}, mix {tuple(mix.shape)}, write {tuple(write.shape)} for "
                          f"{S} streams of {T} x {W}")
    return delta.data_ptr(), mix.data_ptr(), write.data_ptr()


def hc_norm(streams: torch.Tensor, pending, read: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            status: torch.Tensor) -> None:
    """``streams``: float32 [T, S, W].  With ``pending`` = (delta [T, W], mix [S, S] indexed [from, to], write [S])
    the streams are first renewed in place, stream t <- sum_s mix[s, t] stream s + write[t] delta.  Then
    out [T, W] = rmsnorm(sum_s read[s] stream s) * weight."""
    _check("hc_norm.streams", streams, torch.float32)
    _check("hc_norm.read", read, torch.float32)
    _check("hc_norm.weight", weight, torch.float32)
    _check("hc_norm.out", out)
    T, S, W = streams.shape
    if tuple(out.shape) != (T, W) or read.numel() != S or weight.numel() != W:
        raise KernelError(f"hc_norm: streams {tuple(streams.shape)}, out {tuple(out.shape)}, read {tuple(read.shape)}")
    d, m, wr = _hc_pending("hc_norm", pending, T, S, W, out.dtype)
    code = library().q3_hc_norm(streams.data_ptr(), d, m, wr, read.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                dtype_tag(out.dtype), T, S, W, float(eps), status.data_ptr(), _stream())
    _done("hc_norm", code, f"streams {S}")


def hc_sum_norm_rows(streams: torch.Tensor, pending, weight: torch.Tensor, rows: torch.Tensor, out: torch.Tensor,
                     eps: float, status: torch.Tensor) -> None:
    """out [R, W] = rmsnorm(sum of the streams of row rows[r]) * weight, with ``pending`` (see ``hc_norm``)
    applied to those rows first; the streams are left as they are."""
    _check("hc_sum_norm_rows.streams", streams, torch.float32)
    _check("hc_sum_norm_rows.weight", weight, torch.float32)
    _check("hc_sum_norm_rows.rows", rows, torch.int32)
    _check("hc_sum_norm_rows.out", out)
    T, S, W = streams.shape
    R = rows.numel()
    if tuple(out.shape) != (R, W) or weight.numel() != W:
        raise KernelError(f"hc_sum_norm_rows: streams {tuple(streams.shape)}, out {tuple(out.shape)}")
    d, m, wr = _hc_pending("hc_sum_norm_rows", pending, T, S, W, out.dtype)
    code = library().q3_hc_sum_norm_rows(streams.data_ptr(), d, m, wr, weight.data_ptr(), rows.data_ptr(), out.data_ptr(),
                                         dtype_tag(out.dtype), T, R, S, W, float(eps), status.data_ptr(), _stream())
    _done("hc_sum_norm_rows", code, f"streams {S}")


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap), in place (float32)."""
    _check("softcap.logits", logits, torch.float32)
    code = library().q3_softcap(logits.data_ptr(), logits.numel(), float(cap), _stream())
    _done("softcap", code, f"cap {cap}")


def act(x: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out = activation(x), element by element (evaluated in float32); ``out`` may be ``x``."""
    _check("act.x", x)
    _check("act.out", out, x.dtype)
    if out.shape != x.shape:
        raise KernelError(f"act: x {tuple(x.shape)}, out {tuple(out.shape)}")
    code = library().q3_act(x.data_ptr(), out.data_ptr(), dtype_tag(x.dtype), x.numel(), activation_code(activation, gate=True),
                            _stream())
    _done("act", code)


# ------------------------------------------------------------------ attention through a latent
ROTARY_PAIRINGS = {"halves": 0, "neighbours": 1}  # which values of a vector turn together


def rotary_pairing(name: str) -> int:
    if name not in ROTARY_PAIRINGS:
        raise KernelError(f"unknown pairing '{name}' of a rotation (known: {', '.join(ROTARY_PAIRINGS)})")
    return ROTARY_PAIRINGS[name]


def latent_kv_post(proj: torch.Tensor, q_rank: int, kv_col: int, rank: int, rot: int, dims: int, gate_col: int, heads: int,
                   q_norm: torch.Tensor, kv_norm: torch.Tensor, eps: float, freq: torch.Tensor, magnitude: float,
                   positions: torch.Tensor, tok_seq: torch.Tensor, table: torch.Tensor, c_pages: torch.Tensor,
                   r_pages: torch.Tensor, cq: torch.Tensor, gate: Optional[torch.Tensor], write_cache: bool,
                   status: torch.Tensor, pairing: str = "halves") -> None:
    """From one product ``proj`` [T, ld] (query latent at column 0, kv latent and shared key part from ``kv_col``,
    gate pre-activations from ``gate_col``): cq = rmsnorm(query latent) * q_norm; the normed kv latent and the key part
    rotated by position into the pages ``c_pages`` [pages, 1, page, rank] and ``r_pages`` [pages, 1, page, rot];
    gate [T, heads] = sigmoid (float32; None: the mixer has no gates).  The first ``dims`` values of the key part are
    rotated (``pairing`` "halves": pairs i, i + dims / 2; "neighbours": pairs 2i, 2i + 1; angle position * freq[i], sine
    and cosine times ``magnitude``)."""
    _check("latent_kv_post.proj", proj)
    _check("latent_kv_post.cq", cq, proj.dtype)
    _check("latent_kv_post.c_pages", c_pages, proj.dtype)
    _check("latent_kv_post.r_pages", r_pages, proj.dtype)
    if gate is not None:
        _check("latent_kv_post.gate", gate, torch.float32)
    for name, t in (("q_norm", q_norm), ("kv_norm", kv_norm), ("freq", freq)):
        _check(f"latent_kv_post.{name}", t, torch.float32)
    for name, t in (("positions", positions), ("tok_seq", tok_seq), ("table", table)):
        _check(f"latent_kv_post.{name}", t, torch.int32)
    T, ld = proj.shape
    page_size = c_pages.shape[2]
    if (tuple(cq.shape) != (T, q_rank) or (gate is not None and tuple(gate.shape) != (T, heads)) or c_pages.shape[1] != 1
            or c_pages.shape[3] != rank
            or tuple(r_pages.shape) != (c_pages.shape[0], 1, page_size, rot) or q_norm.numel() != q_rank
            or kv_norm.numel() != rank or freq.numel() * 2 != dims or kv_col < q_rank or kv_col + rank + rot > ld
            or (gate is not None and (gate_col < 0 or gate_col + heads > ld)) or positions.numel() != T
            or tok_seq.numel() != T):
        raise KernelError(f"latent_kv_post: proj {tuple(proj.shape)}, cq {tuple(cq.shape)}, c {tuple(c_pages.shape)}, "
                          f"r {tuple(r_pages.shape)}")
    code = library().q3_latent_kv_post(
        proj.data_ptr(), ld, int(q_rank), int(kv_col), int(rank), int(rot), int(dims), int(gate_col), int(heads),
        q_norm.data_ptr(), kv_norm.data_ptr(), float(eps), freq.data_ptr(), float(magnitude), positions.data_ptr(),
        tok_seq.data_ptr(), table.data_ptr(), table.shape[1], page_size, c_pages.shape[0], cq.data_ptr(),
        c_pages.data_ptr(), r_pages.data_ptr(), _ptr(gate), 1 if write_cache else 0, dtype_tag(proj.dtype), T,
        rotary_pairing(pairing), status.data_ptr(), _stream())
    _done("latent_kv_post", code, f"ranks {q_rank}/{rank}, rot {rot}")


def latent_q_post(q: torch.Tensor, heads: int, dim: int, rot: int, dims: int, freq: torch.Tensor, magnitude: float,
                  positions: torch.Tensor, q_plain: torch.Tensor, q_rot: torch.Tensor, pairing: str = "halves") -> None:
    """q [T, heads * (dim + rot)] -> q_plain [T, heads * dim] (as it is) and q_rot [T, heads, rot] (rotated by position)."""
    _check("latent_q_post.q", q)
    _check("latent_q_post.q_plain", q_plain, q.dtype)
    _check("latent_q_post.q_rot", q_rot, q.dtype)
    _check("latent_q_post.freq", freq, torch.float32)
    _check("latent_q_post.positions", positions, torch.int32)
    T = q.shape[0]
    if (q.shape[1] != heads * (dim + rot) or tuple(q_plain.shape) != (T, heads * dim) or tuple(q_rot.shape) != (T, heads, rot)
            or freq.numel() * 2 != dims or positions.numel() != T):
        raise KernelError(f"latent_q_post: q {tuple(q.shape)}, q_plain {tuple(q_plain.shape)}, q_rot {tuple(q_rot.shape)}")
    code = library().q3_latent_q_post(q.data_ptr(), int(heads), int(dim), int(rot), int(dims), freq.data_ptr(),
                                      float(magnitude), positions.data_ptr(), q_plain.data_ptr(), q_rot.data_ptr(),
                                      dtype_tag(q.dtype), T, rotary_pairing(pairing), _stream())
    _done("latent_q_post", code, f"heads {heads} of {dim}+{rot}")


def latent_attn_ref(q_abs: torch.Tensor, q_rot: torch.Tensor, c_pages: torch.Tensor, r_pages: torch.Tensor,
                    positions: torch.Tensor, tok_seq: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float,
                    status: torch.Tensor, sink: Optional[torch.Tensor] = None) -> None:
    """Causal softmax attention over latents: q_abs float32 [H, T, rank] (the plain query taken through the key
    up-projection), q_rot [T, H, rot]; score = (q_abs . c + q_rot . r) * scale over the keys 0 .. position of the
    token's request; out [T, H * rank] = sum_j p_j c_j.  A warp per (token, head), keys one by one.  ``sink``: float32
    [H] or None: head h's weights are exp(s_j) / (sum_j exp(s_j) + exp(sink_h)), the scale on the scores only."""
    _check("latent_attn_ref.q_abs", q_abs, torch.float32)
    _check("latent_attn_ref.q_rot", q_rot)
    _check("latent_attn_ref.c_pages", c_pages, q_rot.dtype)
    _check("latent_attn_ref.r_pages", r_pages, q_rot.dtype)
    _check("latent_attn_ref.out", out, q_rot.dtype)
    for name, t in (("positions", positions), ("tok_seq", tok_seq), ("table", table)):
        _check(f"latent_attn_ref.{name}", t, torch.int32)
    H, T, rank = q_abs.shape
    rot = q_rot.shape[2]
    if sink is not None:
        _check("latent_attn_ref.sink", sink, torch.float32)
    if (tuple(q_rot.shape) != (T, H, rot) or tuple(out.shape) != (T, H * rank) or c_pages.shape[1] != 1
            or c_pages.shape[3] != rank or r_pages.shape[3] != rot or r_pages.shape[:3] != c_pages.shape[:3]
            or (sink is not None and sink.numel() != H)):
        raise KernelError(f"latent_attn_ref: q_abs {tuple(q_abs.shape)}, q_rot {tuple(q_rot.shape)}, c "
                          f"{tuple(c_pages.shape)}, r {tuple(r_pages.shape)}, out {tuple(out.shape)}")
    code = library().q3_latent_attn_ref(q_abs.data_ptr(), q_rot.data_ptr(), c_pages.data_ptr(), r_pages.data_ptr(),
                                        positions.data_ptr(), tok_seq.data_ptr(), table.data_ptr(), table.shape[1],
                                        c_pages.shape[2], c_pages.shape[0], out.data_ptr(), dtype_tag(out.dtype), T, H,
                                        rank, rot, float(scale), _ptr(sink), status.data_ptr(), _stream())
    _done("latent_attn_ref", code, f"heads {H}, rank {rank}, rot {rot}")


def gate_heads(o: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[t, h * dv + v] = o[h, t, v] * gate[t, h]; o float32 [H, T, dv], gate float32 [T, H] (None: no gates, the
    heads are only laid side by side in the compute dtype)."""
    _check("gate_heads.o", o, torch.float32)
    if gate is not None:
        _check("gate_heads.gate", gate, torch.float32)
    _check("gate_heads.out", out)
    H, T, dv = o.shape
    if (gate is not None and tuple(gate.shape) != (T, H)) or tuple(out.shape) != (T, H * dv):
        raise KernelError(f"gate_heads: o {tuple(o.shape)}, out {tuple(out.shape)}")
    code = library().q3_gate_heads(o.data_ptr(), _ptr(gate), out.data_ptr(), dtype_tag(out.dtype), T, H, dv, _stream())
    _done("gate_heads", code)


# ------------------------------------------------------------------ state-space recurrence with a decay per head
def ssd_chunk() -> int:
    """Tokens per chunk of the chunked state-space scan."""
    if "ssd chunk" not in _DEVICE_FACTS:
        _DEVICE_FACTS["ssd chunk"] = int(library()._lib.q3_ssd_chunk())
    return _DEVICE_FACTS["ssd chunk"]


def ssd_scratch_numel(num_tokens: int, num_seqs: int, heads: int, vdim: int, n_state: int) -> int:
    """Floats of scratch that the chunked form needs for a step of so many tokens and requests."""
    record = int(library()._lib.q3_ssd_record_floats(heads, vdim, n_state))
    if ssd_matrix_form(vdim, n_state):
        record = max(record, int(library()._lib.q3_ssd_mma_record_floats(heads, vdim, n_state)))
    return (num_tokens // ssd_chunk() + num_seqs + 1) * record


def ssd_matrix_form(vdim: int, n_state: int) -> bool:
    """Whether chunks of these sizes run as matrix products on the tensor cores (heads of 64 channels, a state of 64
    or 128); other sizes walk their chunks token by token."""
    return bool(library()._lib.q3_ssd_mma_takes(int(vdim), int(n_state)))


def ssd_chunked_pays(dtype: torch.dtype, max_q_len: int) -> bool:
    """bfloat16 with a portion of at least four chunks: the portions run in chunks side by side.  The float32 run
    walks every portion in one piece, so that its bits do not depend on how a prompt was cut."""
    return dtype == torch.bfloat16 and max_q_len >= 4 * ssd_chunk()


def ssd_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
             d_skip: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, slot_ids: torch.Tensor, num_seqs: int,
             y: torch.Tensor, heads: int, vdim: int, n_state: int, groups: int, status: torch.Tensor,
             max_q_len: int = 0, scratch: Optional[torch.Tensor] = None, kernel: str = "auto") -> None:
    """Per head h (group g = h // (heads / groups)): step = softplus(dt + dt_bias[h]); S <- exp(-exp(a_log[h]) step) S
    + step B_g x_h^T; y_h = S^T C_g + d_skip[h] x_h.  xbc [T, ld]: x (heads * vdim columns), then B and C (groups *
    n_state each); dt: proj[:, dt_col + h]; state float32 [slots, heads, n_state, vdim]; y float32 [T, heads * vdim].
    With ``scratch`` (``ssd_scratch_numel`` floats) and a longest portion ``max_q_len`` of ``ssd_chunked_pays`` the
    portions are cut into chunks that run side by side: as matrix products on the tensor cores where
    ``ssd_matrix_form`` takes the sizes (``kernel="walk"`` keeps the token-by-token walk of the chunks)."""
    _check("ssd_scan.xbc", xbc)
    _check("ssd_scan.proj", proj, xbc.dtype)
    _check("ssd_scan.y", y, torch.float32)
    _check("ssd_scan.state", state, torch.float32)
    for name, t in (("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip)):
        _check(f"ssd_scan.{name}", t, torch.float32)
        if t.numel() != heads:
            raise KernelError(f"ssd_scan: {name} has {t.numel()} values for {heads} heads")
    T, ld = xbc.shape
    inner = heads * vdim
    if (ld != inner + 2 * groups * n_state or tuple(y.shape) != (T, inner) or proj.shape[0] != T or dt_col < 0
            or dt_col + heads > proj.shape[1] or tuple(state.shape[1:]) != (heads, n_state, vdim)
            or q_start.numel() < num_seqs + 1):
        raise KernelError(f"ssd_scan: xbc {tuple(xbc.shape)}, proj {tuple(proj.shape)}, y {tuple(y.shape)}, state "
                          f"{tuple(state.shape)}")
    chunked = scratch is not None and ssd_chunked_pays(xbc.dtype, max_q_len)
    if chunked:
        _check("ssd_scan.scratch", scratch, torch.float32)
        if scratch.numel() < ssd_scratch_numel(T, num_seqs, heads, vdim, n_state):
            raise KernelError(f"ssd_scan: scratch of {scratch.numel()} floats for {T} tokens of {num_seqs} requests")
    if chunked and kernel != "walk" and ssd_matrix_form(vdim, n_state) and ld % 8 == 0:
        code = library().q3_ssd_scan_mma(xbc.data_ptr(), ld, proj.data_ptr(), proj.shape[1], int(dt_col),
                                         dt_bias.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(),
                                         scratch.data_ptr(), q_start.data_ptr(), slot_ids.data_ptr(), y.data_ptr(), T,
                                         int(num_seqs), int(max_q_len), heads, vdim, n_state, groups, state.shape[0],
                                         _stream())
        _done("ssd_scan (matrix form)", code, f"heads {heads} x {vdim}, state {n_state}, groups {groups}")
        return
    code = library().q3_ssd_scan(xbc.data_ptr(), ld, proj.data_ptr(), proj.shape[1], int(dt_col), dt_bias.data_ptr(),
                                 a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), _ptr(scratch) if chunked else None,
                                 q_start.data_ptr(), slot_ids.data_ptr(), y.data_ptr(), dtype_tag(xbc.dtype), T,
                                 int(num_seqs), int(max_q_len), heads, vdim, n_state, groups, state.shape[0],
                                 status.data_ptr(), _stream())
    _done("ssd_scan", code, f"heads {heads} x {vdim}, state {n_state}, groups {groups}")


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, z_col: int, weight: torch.Tensor, out: torch.Tensor, parts: int,
                     eps: float) -> None:
    """out = unit_rms_per_part(y * silu(z)) * weight: the row of I values is cut into ``parts`` equal parts, each divided
    by its own root mean square.  y float32 [T, I]; z = z[:, z_col : z_col + I]."""
    _check("gated_group_norm.y", y, torch.float32)
    _check("gated_group_norm.z", z)
    _check("gated_group_norm.out", out, z.dtype)
    _check("gated_group_norm.weight", weight, torch.float32)
    T, I = y.shape
    if tuple(out.shape) != (T, I) or z.shape[0] != T or z_col < 0 or z_col + I > z.shape[1] or weight.numel() != I:
        raise KernelError(f"gated_group_norm: y {tuple(y.shape)}, z {tuple(z.shape)}, out {tuple(out.shape)}")
    code = library().q3_gated_group_norm(y.data_ptr(), z.data_ptr(), z.shape[1], int(z_col), weight.data_ptr(),
                                         out.data_ptr(), dtype_tag(out.dtype), T, I, int(parts), float(eps), _stream())
    _done("gated_group_norm", code, f"{parts} parts of {I}")


LATENT_MAX_SPLITS = 32  # key ranges per request of the single-token form
LATENT_SPLIT_TILES = 4   # a range is at least so many times 32 keys


def latent_attention_fast(dtype: torch.dtype, rank: int, rot: int) -> bool:
    """Whether the tensor-core kernel takes this latent: bfloat16, a latent of 64, 128, 256 or 512 values."""
    return dtype == torch.bfloat16 and bool(library()._lib.q3_latent_attn_mma_takes(int(rank), int(rot)))


def latent_partial_numel(num_seqs: int, heads: int, rank: int) -> int:
    """Floats of scratch that the single-token form needs for its key ranges."""
    return num_seqs * heads * LATENT_MAX_SPLITS * (rank + 2)


def latent_decode_splits(num_seqs: int, heads: int, max_kv_len: int) -> int:
    """Key ranges per request when every row brings one token.  A block takes about 1.6 us per 16-key tile whatever
    else runs (its tile's latency and a chain of dependent steps), and every range costs the merge a pass: as many
    ranges as fill the four places an SM has for these blocks, none shorter than ``LATENT_SPLIT_TILES`` x 32 keys
    (measured: 8 requests over 2,048 keys 211 us in one range, 44 in 16; 64 requests 71 us in 8 ranges, 93 in 16;
    8 requests over 16,384 keys 128 us in 16 ranges, 99 in 32)."""
    blocks = num_seqs * -(-heads // 16)
    by_length = max(1, -(-max_kv_len // 32) // LATENT_SPLIT_TILES)
    return max(1, min(LATENT_MAX_SPLITS, by_length, 4 * sm_count() // blocks))


def latent_attention(q_abs: torch.Tensor, q_rot: torch.Tensor, c_pages: torch.Tensor, r_pages: torch.Tensor, ctx,
                     table: torch.Tensor, out: torch.Tensor, scale: float, status: torch.Tensor,
                     partial: Optional[torch.Tensor] = None, kernel: str = "auto", sink: Optional[torch.Tensor] = None) -> None:
    """Attention over latents for one step's batch (``ctx``: its positions, rows and lengths): see ``latent_attn_ref``
    for the arithmetic.  bfloat16 with a latent that ``latent_attention_fast`` takes runs on the tensor cores (rows of
    (token, head) pairs over shared key tiles; with ``partial`` and a step of single tokens the keys of a request are
    cut into ranges that run side by side and are merged); everything else, and float32, on the plain kernel.
    ``kernel``: "auto", "plain" or "mma"."""
    H, T, rank = q_abs.shape
    rot = q_rot.shape[2]
    fast = kernel != "plain" and latent_attention_fast(q_rot.dtype, rank, rot)
    if kernel == "mma" and not fast:
        raise KernelSizeError(f"latent_attention: the tensor-core kernel does not take rank {rank}, rot {rot}, {q_rot.dtype}")
    if not fast:
        latent_attn_ref(q_abs, q_rot, c_pages, r_pages, ctx.positions, ctx.tok_seq, table, out, scale, status, sink=sink)
        return
    if sink is not None:
        _check("latent_attention.sink", sink, torch.float32)
        if sink.numel() != H:
            raise KernelError(f"latent_attention: {sink.numel()} sinks for {H} heads")
    _check("latent_attention.q_abs", q_abs, torch.float32)
    _check("latent_attention.q_rot", q_rot, torch.bfloat16)
    _check("latent_attention.c_pages", c_pages, torch.bfloat16)
    _check("latent_attention.r_pages", r_pages, torch.bfloat16)
    _check("latent_attention.out", out, torch.bfloat16)
    if (tuple(q_rot.shape) != (T, H, rot) or tuple(out.shape) != (T, H * rank) or c_pages.shape[1] != 1
            or c_pages.shape[3] != rank or r_pages.shape[3] != rot or r_pages.shape[:3] != c_pages.shape[:3]):
        raise KernelError(f"latent_attention: q_abs {tuple(q_abs.shape)}, q_rot {tuple(q_rot.shape)}, c "
                          f"{tuple(c_pages.shape)}, r {tuple(r_pages.shape)}, out {tuple(out.shape)}")
    splits = 1
    if ctx.max_q_len == 1 and partial is not None:
        splits = latent_decode_splits(ctx.num_seqs, H, ctx.max_kv_len)
        if partial.numel() < T * H * splits * (rank + 2):
            splits = 1
    code = library().q3_latent_attn_mma(
        q_abs.data_ptr(), q_rot.data_ptr(), c_pages.data_ptr(), r_pages.data_ptr(), ctx.q_start.data_ptr(),
        ctx.kv_len.data_ptr(), table.data_ptr(), table.shape[1], c_pages.shape[2], c_pages.shape[0], out.data_ptr(),
        _ptr(partial) if splits > 1 else None, T, ctx.num_seqs, ctx.max_q_len, H, rank, rot, float(scale), splits,
        _ptr(sink), status.data_ptr(), _stream())
    _done("latent_attention (mma)", code, f"heads {H}, rank {rank}, rot {rot}, splits {splits}")


# ------------------------------------------------------------------ layer norm and the convolution before a sub-layer
def add_layernorm(stream: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: torch.Tensor,
                  out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """stream (float32 [T, W]) += delta in place, then out = (x - mean) / sqrt(var + eps) * weight + bias with var
    the mean of the squared deviations; ``out`` is float32 or the dtype of ``delta``.  With ``rows`` (int32) the
    chosen rows are normed into ``out`` [len(rows), W] and the stream is left as it is."""
    _check("add_layernorm.stream", stream, torch.float32)
    _check("add_layernorm.weight", weight, torch.float32)
    _check("add_layernorm.bias", bias, torch.float32)
    _check("add_layernorm.out", out)
    T, W = stream.shape
    n = T if rows is None else rows.numel()
    dtype = out.dtype if delta is None else delta.dtype
    if delta is not None:
        _check("add_layernorm.delta", delta)
    if rows is not None:
        _check("add_layernorm.rows", rows, torch.int32)
    if (tuple(out.shape) != (n, W) or weight.numel() != W or bias.numel() != W or out.dtype not in (torch.float32, dtype)
            or (delta is not None and tuple(delta.shape) != (T, W))):
        raise KernelError(f"add_layernorm: stream {tuple(stream.shape)}, delta "
                          f"{None if delta is None else tuple(delta.shape)}, out {tuple(out.shape)} {out.dtype}")
    code = library().q3_add_layernorm(stream.data_ptr(), _ptr(delta), weight.data_ptr(), bias.data_ptr(), out.data_ptr(),
                                      1 if out.dtype == torch.float32 else 0, dtype_tag(dtype), _ptr(rows), n, W, float(eps),
                                      _stream())
    _done("add_layernorm", code, f"width {W}")


INPUT_CONV_MAX_TAPS = 16  # the kernel keeps a request's tail in registers while it renews it


def stream_concat(stream: torch.Tensor, delta: Optional[torch.Tensor], other: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [stream[t] + delta[t] | other[t]]: two float32 [T, W] tensors side by side in the dtype of ``out``
    [T, 2 W]; ``delta`` (in that dtype, or None) is added to the first on the way."""
    _check("stream_concat.stream", stream, torch.float32)
    _check("stream_concat.other", other, torch.float32)
    _check("stream_concat.out", out)
    T, W = stream.shape
    if delta is not None:
        _check("stream_concat.delta", delta, out.dtype)
    if (tuple(other.shape) != (T, W) or tuple(out.shape) != (T, 2 * W)
            or (delta is not None and tuple(delta.shape) != (T, W))):
        raise KernelError(f"stream_concat: stream {tuple(stream.shape)}, other {tuple(other.shape)}, out {tuple(out.shape)}")
    code = library().q3_stream_concat(stream.data_ptr(), _ptr(delta), other.data_ptr(), out.data_ptr(), dtype_tag(out.dtype),
                                      T, W, _stream())
    _done("stream_concat", code, f"width {W}")


def add_layernorm_conv1(stream: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: torch.Tensor,
                        conv_weight: torch.Tensor, state: Optional[torch.Tensor], tok_seq: torch.Tensor,
                        slot_ids: torch.Tensor, out: torch.Tensor, eps: float, status: torch.Tensor) -> None:
    """``add_layernorm`` and ``input_conv`` in one launch for a step in which every request brings one token:
    stream += delta, h = layer norm of the row, out = h + conv(h) from the request's state, which is renewed."""
    _check("add_layernorm_conv1.stream", stream, torch.float32)
    _check("add_layernorm_conv1.out", out)
    for name, t in (("weight", weight), ("bias", bias), ("conv_weight", conv_weight)):
        _check(f"add_layernorm_conv1.{name}", t, torch.float32)
    for name, t in (("tok_seq", tok_seq), ("slot_ids", slot_ids)):
        _check(f"add_layernorm_conv1.{name}", t, torch.int32)
    T, W = stream.shape
    K = conv_weight.shape[1]
    if delta is not None:
        _check("add_layernorm_conv1.delta", delta, out.dtype)
    if state is not None:
        _check("add_layernorm_conv1.state", state, torch.float32)
    if (tuple(out.shape) != (T, W) or weight.numel() != W or bias.numel() != W or conv_weight.shape[0] != W
            or (delta is not None and delta.shape != stream.shape) or (K > 1 and (state is None or state.dim() != 3
            or state.shape[1] != K - 1 or state.shape[2] != W))):
        raise KernelError(f"add_layernorm_conv1: stream {tuple(stream.shape)}, out {tuple(out.shape)}, taps "
                          f"{tuple(conv_weight.shape)}, state {None if state is None else tuple(state.shape)}")
    code = library().q3_add_layernorm_conv1(stream.data_ptr(), _ptr(delta), weight.data_ptr(), bias.data_ptr(),
                                            conv_weight.data_ptr(), _ptr(state), tok_seq.data_ptr(), slot_ids.data_ptr(),
                                            out.data_ptr(), dtype_tag(out.dtype), T, W, K,
                                            state.shape[0] if state is not None else 0, float(eps), status.data_ptr(),
                                            _stream())
    _done("add_layernorm_conv1", code, f"width {W}, taps {K}")


def input_conv(h: torch.Tensor, weight: torch.Tensor, state: Optional[torch.Tensor], q_start: torch.Tensor,
               tok_seq: torch.Tensor, slot_ids: torch.Tensor, num_seqs: int, out: torch.Tensor, status: torch.Tensor,
               renew_state: bool = True) -> None:
    """out[t, c] = h[t, c] + sum_j weight[c, j] h[t - (K - 1) + j, c] within each request, h float32 [T, C]; what lies
    before a portion comes from ``state`` (float32 [slots, K - 1, C], zero for a new request; None for K = 1), which is
    renewed afterwards."""
    _check("input_conv.h", h, torch.float32)
    _check("input_conv.weight", weight, torch.float32)
    _check("input_conv.out", out)
    for name, t in (("q_start", q_start), ("tok_seq", tok_seq), ("slot_ids", slot_ids)):
        _check(f"input_conv.{name}", t, torch.int32)
    T, C = h.shape
    K = weight.shape[1]
    if tuple(out.shape) != (T, C) or weight.shape[0] != C or tok_seq.numel() != T or q_start.numel() < num_seqs + 1:
        raise KernelError(f"input_conv: h {tuple(h.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    slots = 0
    if K > 1:
        _check("input_conv.state", state, torch.float32)
        if state.dim() != 3 or tuple(state.shape[1:]) != (K - 1, C):
            raise KernelError(f"input_conv: state {tuple(state.shape)} for {K} taps and {C} channels")
        slots = state.shape[0]
    code = library().q3_input_conv(h.data_ptr(), weight.data_ptr(), _ptr(state) if K > 1 else None, q_start.data_ptr(),
                                   tok_seq.data_ptr(), slot_ids.data_ptr(), out.data_ptr(), dtype_tag(out.dtype), T,
                                   int(num_seqs), C, K, slots, 1 if renew_state else 0, status.data_ptr(), _stream())
    _done("input_conv", code, f"channels {C}, taps {K}")


# ------------------------------------------------------------------ windowed attention over pooled blocks
def _pw_pages(name: str, k_pages, v_pages, pk_pages, pv_pages, dtype):
    for n, t in (("k_pages", k_pages), ("v_pages", v_pages), ("pk_pages", pk_pages), ("pv_pages", pv_pages)):
        _check(f"{name}.{n}", t, dtype)
    if (k_pages.dim() != 4 or v_pages.shape[:3] != k_pages.shape[:3] or pk_pages.shape[1:] != k_pages.shape[1:]
            or pv_pages.shape[1:] != v_pages.shape[1:] or pk_pages.shape[0] != pv_pages.shape[0]):
        raise KernelError(f"{name}: pages k {tuple(k_pages.shape)}, v {tuple(v_pages.shape)}, pooled k "
                          f"{tuple(pk_pages.shape)}, pooled v {tuple(pv_pages.shape)}")


def pw_qkv_post(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, heads: int, kv_heads: int, dim: int, vdim: int,
                q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float, dims: int, freq: torch.Tensor,
                magnitude: float, positions: torch.Tensor, tok_seq: torch.Tensor, table: torch.Tensor, q_out: torch.Tensor,
                k_pages: torch.Tensor, v_pages: torch.Tensor, write_cache: bool, status: torch.Tensor) -> None:
    """From one product ``proj`` [T, ld] (q at column ``q_col``, k at ``k_col``, v at ``v_col``): RMS norm of the whole q and of
    the whole k projection (weights ``q_norm`` [heads * dim], ``k_norm`` [kv_heads * dim]), rotation of the first
    ``dims`` values of every head by position * freq (sines and cosines times ``magnitude``), q to ``q_out``
    [T, heads, dim], k and v into their pages.  Without norm weights (both None) q and k are rotated as projected."""
    _check("pw_qkv_post.proj", proj)
    if (q_norm is None) != (k_norm is None):
        raise KernelError("pw_qkv_post: norm weights for both q and k, or for neither")
    _check("pw_qkv_post.q_out", q_out, proj.dtype)
    _check("pw_qkv_post.k_pages", k_pages, proj.dtype)
    _check("pw_qkv_post.v_pages", v_pages, proj.dtype)
    for name, t in (("q_norm", q_norm), ("k_norm", k_norm), ("freq", freq)):
        if t is not None:
            _check(f"pw_qkv_post.{name}", t, torch.float32)
    for name, t in (("positions", positions), ("tok_seq", tok_seq), ("table", table)):
        _check(f"pw_qkv_post.{name}", t, torch.int32)
    T, ld = proj.shape
    if (tuple(q_out.shape) != (T, heads, dim)
            or (q_norm is not None and (q_norm.numel() != heads * dim or k_norm.numel() != kv_heads * dim))
            or freq.numel() < dims // 2 or k_col + kv_heads * dim > ld or v_col + kv_heads * vdim > ld
            or q_col < 0 or q_col + heads * dim > ld or k_col < 0 or v_col < 0
            or tuple(k_pages.shape[1:]) != (kv_heads, k_pages.shape[2], dim)
            or tuple(v_pages.shape) != (k_pages.shape[0], kv_heads, k_pages.shape[2], vdim)):
        raise KernelError(f"pw_qkv_post: proj {tuple(proj.shape)}, q_out {tuple(q_out.shape)}, k pages "
                          f"{tuple(k_pages.shape)}, v pages {tuple(v_pages.shape)}")
    code = library().q3_pw_qkv_post(proj.data_ptr() + int(q_col) * proj.element_size(), ld, int(k_col) - int(q_col),
                                    int(v_col) - int(q_col), heads, kv_heads, dim, vdim, _ptr(q_norm),
                                    _ptr(k_norm), float(eps), int(dims), freq.data_ptr(), float(magnitude),
                                    positions.data_ptr(), tok_seq.data_ptr(), table.data_ptr(), table.shape[1],
                                    k_pages.shape[2], k_pages.shape[0], q_out.data_ptr(), k_pages.data_ptr(),
                                    v_pages.data_ptr(), 1 if write_cache else 0, dtype_tag(proj.dtype), T, status.data_ptr(),
                                    _stream())
    _done("pw_qkv_post", code, f"heads {heads}/{kv_heads}, dim {dim}, vdim {vdim}, rotated {dims}")


def pool_blocks(k_pages: torch.Tensor, v_pages: torch.Tensor, pk_pages: torch.Tensor, pv_pages: torch.Tensor,
                q_start: torch.Tensor, kv_len: torch.Tensor, table: torch.Tensor, ptable: torch.Tensor, num_seqs: int,
                max_q_len: int, pool: int, status: torch.Tensor) -> None:
    """For every block of ``pool`` tokens whose last token is one of this step's: the mean of its keys and of its values
    (as the token pages hold them) into entry ``block index`` of the block pages."""
    _pw_pages("pool_blocks", k_pages, v_pages, pk_pages, pv_pages, k_pages.dtype)
    for name, t in (("q_start", q_start), ("kv_len", kv_len), ("table", table), ("ptable", ptable)):
        _check(f"pool_blocks.{name}", t, torch.int32)
    max_blocks = (int(max_q_len) + pool - 1) // pool + 1
    code = library().q3_pool_blocks(k_pages.data_ptr(), v_pages.data_ptr(), pk_pages.data_ptr(), pv_pages.data_ptr(),
                                    q_start.data_ptr(), kv_len.data_ptr(), table.data_ptr(), table.shape[1], k_pages.shape[0],
                                    ptable.data_ptr(), ptable.shape[1], pk_pages.shape[0], k_pages.shape[2], k_pages.shape[1],
                                    k_pages.shape[3], v_pages.shape[3], int(pool), int(num_seqs), max_blocks,
                                    dtype_tag(k_pages.dtype), status.data_ptr(), _stream())
    _done("pool_blocks", code, f"pool {pool}")


def pw_attn_ref(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, pk_pages: torch.Tensor,
                pv_pages: torch.Tensor, positions: torch.Tensor, tok_seq: torch.Tensor, table: torch.Tensor,
                ptable: torch.Tensor, out: torch.Tensor, window: int, pool: int, scale: float, softcap: Optional[float],
                out_scale: float, status: torch.Tensor, block_limit: int = -1) -> None:
    """Softmax attention of q [T, H, D] over the last ``window`` tokens and the pooled blocks before them (with
    ``block_limit`` >= 0 only the first so many blocks are ever read: with blocks of one token whose pages are the
    token pages themselves, that is a window that also keeps a request's first tokens); head h's
    result times ``out_scale`` goes to columns h * vdim .. of ``out`` (rows of any pitch: a column view of a wider
    buffer is taken).  A warp per (token, head), float32 arithmetic, keys one by one."""
    _check("pw_attn_ref.q", q)
    _pw_pages("pw_attn_ref", k_pages, v_pages, pk_pages, pv_pages, q.dtype)
    for name, t in (("positions", positions), ("tok_seq", tok_seq), ("table", table), ("ptable", ptable)):
        _check(f"pw_attn_ref.{name}", t, torch.int32)
    T, H, D = q.shape
    G, Dv = k_pages.shape[1], v_pages.shape[3]
    if (out.dtype != q.dtype or out.dim() != 2 or out.shape[0] != T or out.shape[1] != H * Dv or out.stride(1) != 1
            or k_pages.shape[3] != D or not out.is_cuda):
        raise KernelError(f"pw_attn_ref: q {tuple(q.shape)}, k pages {tuple(k_pages.shape)}, out {tuple(out.shape)} "
                          f"strides {out.stride()}")
    code = library().q3_pw_attn_ref(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), pk_pages.data_ptr(),
                                    pv_pages.data_ptr(), positions.data_ptr(), tok_seq.data_ptr(), table.data_ptr(),
                                    table.shape[1], k_pages.shape[0], ptable.data_ptr(), ptable.shape[1], pk_pages.shape[0],
                                    k_pages.shape[2], out.data_ptr(), out.stride(0), dtype_tag(q.dtype), T, H, G, D, Dv,
                                    int(window), int(pool), float(scale), float(softcap or 0.0), float(out_scale),
                                    int(block_limit), status.data_ptr(), _stream())
    _done("pw_attn_ref", code, f"heads {H}/{G}, dim {D}, vdim {Dv}")


def pw_attention_fast(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    """Whether the tensor-core kernel takes these heads: bfloat16, keys and values of 32, 64 or 128 values."""
    return dtype == torch.bfloat16 and bool(library()._lib.q3_pw_attn_mma_takes(int(dim), int(vdim)))


def pw_attn_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, pk_pages: torch.Tensor,
                pv_pages: torch.Tensor, ctx, table: torch.Tensor, ptable: torch.Tensor, out: torch.Tensor, window: int,
                pool: int, scale: float, softcap: Optional[float], out_scale: float, status: torch.Tensor,
                partial: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, block_limit: int = -1) -> None:
    """The same attention as ``pw_attn_ref`` on the tensor cores (bfloat16): tiles of 64 entries of the block pages
    and of the token pages in one online softmax, 128 (token, head) rows of one kv head to a block.  ``partial``
    (``pw_attn_partial``): scratch with which a step of single tokens cuts every request's keys into ranges that run
    side by side and are merged in ascending order."""
    _check("pw_attn_mma.q", q, torch.bfloat16)
    _pw_pages("pw_attn_mma", k_pages, v_pages, pk_pages, pv_pages, q.dtype)
    for name, t in (("q_start", ctx.q_start), ("kv_len", ctx.kv_len), ("table", table), ("ptable", ptable)):
        _check(f"pw_attn_mma.{name}", t, torch.int32)
    T, H, D = q.shape
    G, Dv = k_pages.shape[1], v_pages.shape[3]
    if (out.dtype != q.dtype or out.dim() != 2 or out.shape[0] != T or out.shape[1] != H * Dv or out.stride(1) != 1
            or k_pages.shape[3] != D or not out.is_cuda):
        raise KernelError(f"pw_attn_mma: q {tuple(q.shape)}, k pages {tuple(k_pages.shape)}, out {tuple(out.shape)} "
                          f"strides {out.stride()}")
    part_o = part_ml = None
    part_rows = 0
    if partial is not None:
        part_o, part_ml = partial
        _check("pw_attn_mma.partial", part_o, torch.float32)
        _check("pw_attn_mma.partial", part_ml, torch.float32)
        part_rows = min(part_o.numel() // Dv, part_ml.numel() // 2)
    code = library().q3_pw_attn_mma(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), pk_pages.data_ptr(),
                                    pv_pages.data_ptr(), out.data_ptr(), out.stride(0), ctx.q_start.data_ptr(),
                                    ctx.kv_len.data_ptr(), table.data_ptr(), table.shape[1], k_pages.shape[0],
                                    ptable.data_ptr(), ptable.shape[1], pk_pages.shape[0], k_pages.shape[2], ctx.num_seqs,
                                    ctx.max_q_len, H, G, D, Dv, float(scale), float(softcap or 0.0), float(out_scale),
                                    int(window), int(pool), int(block_limit), T, _ptr(part_o), _ptr(part_ml), part_rows,
                                    status.data_ptr(), _stream())
    _done("pw_attn_mma", code, f"heads {H}/{G}, dim {D}, vdim {Dv}")


PW_ATTN_MAX_RANGES = 32  # the most ranges that the keys of a request are cut into


def pw_attn_partial(alloc, max_seqs: int, heads: int, vdim: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scratch for ``pw_attn_mma``: room for the most ranges for a step of ``max_seqs`` single tokens (a step of more
    tokens gets fewer ranges)."""
    rows = max_seqs * heads * PW_ATTN_MAX_RANGES
    return (alloc("pwattn.partial_o", rows * vdim, dtype=torch.float32),
            alloc("pwattn.partial_ml", rows * 2, dtype=torch.float32))


def pooled_window_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, pk_pages: torch.Tensor,
                            pv_pages: torch.Tensor, ctx, table: torch.Tensor, ptable: torch.Tensor, out: torch.Tensor,
                            window: int, pool: int, scale: float, softcap: Optional[float], out_scale: float,
                            status: torch.Tensor, partial: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                            block_limit: int = -1) -> None:
    """The attention of a step's batch over windows and pooled blocks, by the kernel that suits dtype and shape: the
    tensor-core kernel for bfloat16 heads it takes (an output whose rows and start allow paired stores), the plain
    one for everything else."""
    if (pw_attention_fast(q.dtype, q.shape[2], v_pages.shape[3]) and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0):
        pw_attn_mma(q, k_pages, v_pages, pk_pages, pv_pages, ctx, table, ptable, out, window, pool, scale, softcap,
                    out_scale, status, partial, block_limit)
    else:
        pw_attn_ref(q, k_pages, v_pages, pk_pages, pv_pages, ctx.positions, ctx.tok_seq, table, ptable, out, window, pool,
                    scale, softcap, out_scale, status, block_limit)


# ------------------------------------------------------------------ a recurrence gated by the current token alone
def mingru_chunk() -> int:
    """Tokens per chunk of the chunked minGRU scan."""
    if "mingru chunk" not in _DEVICE_FACTS:
        _DEVICE_FACTS["mingru chunk"] = int(library()._lib.q3_mingru_chunk())
    return _DEVICE_FACTS["mingru chunk"]


def mingru_scratch_numel(num_tokens: int, num_seqs: int, channels: int) -> int:
    """Floats of scratch that the chunked minGRU scan needs for a step of so many tokens and requests."""
    return (num_tokens // mingru_chunk() + num_seqs + 1) * 2 * channels


def mingru_chunked_pays(dtype: torch.dtype, max_q_len: int) -> bool:
    """Whether a step whose longest portion has ``max_q_len`` tokens goes to the chunked scan: the bfloat16 run, from
    four chunks on (the float32 run keeps the single walk, whose bits do not depend on the cut)."""
    return dtype == torch.bfloat16 and max_q_len >= 4 * mingru_chunk()


def mingru_scan(proj: torch.Tensor, z_col: int, u_col: int, g_col: int, z_bias: torch.Tensor, u_bias: torch.Tensor,
                state: torch.Tensor, q_start: torch.Tensor, slot_ids: torch.Tensor, num_seqs: int, out: torch.Tensor,
                out_scale: float, status: torch.Tensor, max_q_len: int = 0, scratch: Optional[torch.Tensor] = None) -> None:
    """z = sigmoid(proj[:, z_col..] + z_bias), u = proj[:, u_col..] + u_bias, candidate = u + 1/2 (u >= 0) or sigmoid(u);
    S <- (1 - z) S + z candidate per request, token by token (``state`` float32 [slots, C]);
    out = S * silu(proj[:, g_col..]) * out_scale.  ``out``: [T, C], rows of any pitch.  With ``scratch`` (float32,
    ``mingru_scratch_numel``) and a longest portion ``max_q_len`` of ``mingru_chunked_pays`` the portions are cut
    into chunks that run side by side."""
    _check("mingru_scan.proj", proj)
    _check("mingru_scan.state", state, torch.float32)
    for name, t in (("z_bias", z_bias), ("u_bias", u_bias)):
        _check(f"mingru_scan.{name}", t, torch.float32)
    for name, t in (("q_start", q_start), ("slot_ids", slot_ids)):
        _check(f"mingru_scan.{name}", t, torch.int32)
    T, ld = proj.shape
    C = state.shape[1]
    if (out.dtype != proj.dtype or out.dim() != 2 or tuple(out.shape) != (T, C) or out.stride(1) != 1 or state.dim() != 2
            or z_bias.numel() != C or u_bias.numel() != C or max(z_col, u_col, g_col) + C > ld or min(z_col, u_col, g_col) < 0):
        raise KernelError(f"mingru_scan: proj {tuple(proj.shape)}, columns {z_col}, {u_col}, {g_col}, state "
                          f"{tuple(state.shape)}, out {tuple(out.shape)}")
    if scratch is not None and mingru_chunked_pays(proj.dtype, max_q_len):
        _check("mingru_scan.scratch", scratch, torch.float32)
        if scratch.numel() < mingru_scratch_numel(T, num_seqs, C):
            raise KernelError(f"mingru_scan: scratch of {scratch.numel()} floats for {T} tokens of {num_seqs} requests")
        code = library().q3_mingru_scan_chunked(
            proj.data_ptr(), ld, int(z_col), int(u_col), int(g_col), z_bias.data_ptr(), u_bias.data_ptr(), state.data_ptr(),
            scratch.data_ptr(), q_start.data_ptr(), slot_ids.data_ptr(), out.data_ptr(), out.stride(0),
            dtype_tag(proj.dtype), T, int(num_seqs), int(max_q_len), C, state.shape[0], float(out_scale), status.data_ptr(),
            _stream())
        _done("mingru_scan_chunked", code, f"channels {C}")
        return
    code = library().q3_mingru_scan(proj.data_ptr(), ld, int(z_col), int(u_col), int(g_col), z_bias.data_ptr(),
                                    u_bias.data_ptr(), state.data_ptr(), q_start.data_ptr(), slot_ids.data_ptr(),
                                    out.data_ptr(), out.stride(0), dtype_tag(proj.dtype), T, int(num_seqs), C, state.shape[0],
                                    float(out_scale), status.data_ptr(), _stream())
    _done("mingru_scan", code, f"channels {C}")


# ------------------------------------------------------------------ routed experts
MOE_MAX_TOP = 32  # experts per token that the routing kernel lists


def moe_route(h: torch.Tensor, router: torch.Tensor, bias: Optional[torch.Tensor], ids: torch.Tensor, weights: torch.Tensor,
              scale: float) -> None:
    """Scores s = sigmoid(h router^T) in float32; ``ids`` [T, top] the experts with the largest s + bias, ``weights``
    [T, top] their s * scale."""
    _check("moe_route.h", h)
    _check("moe_route.router", router, torch.float32)
    _check("moe_route.ids", ids, torch.int32)
    _check("moe_route.weights", weights, torch.float32)
    T, W = h.shape
    E = router.shape[0]
    top = ids.shape[1]
    if bias is not None:
        _check("moe_route.bias", bias, torch.float32)
    if (router.shape[1] != W or tuple(ids.shape) != (T, top) or tuple(weights.shape) != (T, top)
            or (bias is not None and bias.numel() != E)):
        raise KernelError(f"moe_route: h {tuple(h.shape)}, router {tuple(router.shape)}, ids {tuple(ids.shape)}")
    code = library().q3_moe_route(h.data_ptr(), router.data_ptr(), _ptr(bias), ids.data_ptr(), weights.data_ptr(),
                                  dtype_tag(h.dtype), T, W, E, top, float(scale), _stream())
    _done("moe_route", code, f"experts {E}, top {top}")


def moe_pairs(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
              base: Optional[torch.Tensor], act_buf: torch.Tensor, out: torch.Tensor, activation: str,
              gate_block: int = 0, in_weights: Optional[torch.Tensor] = None) -> None:
    """out[t] = base[t] + sum_k weights[t, k] down[ids[t, k]] act(up[ids[t, k]] h[t]); up [E, F, W], down [E, W, F];
    ``act_buf`` [T * top, F] receives the activations.  Every (token, expert) pair streams its expert once.
    ``gate_block`` > 0: gated experts, act(gate h) * (up h), ``up`` being [E, 2 F, W] with gate and up rows alternating
    in blocks of so many rows.  ``in_weights`` [T, top]: what multiplies the expert's input (``weights`` still
    multiply its output: ones, for a design that weighs the input only)."""
    _check("moe_pairs.h", h)
    for name, t in (("up", up), ("down", down), ("act_buf", act_buf), ("out", out)):
        _check(f"moe_pairs.{name}", t, h.dtype)
    _check("moe_pairs.ids", ids, torch.int32)
    _check("moe_pairs.weights", weights, torch.float32)
    T, W = h.shape
    E, F = up.shape[0], up.shape[1] // (2 if gate_block else 1)
    top = ids.shape[1]
    if base is not None:
        _check("moe_pairs.base", base, h.dtype)
    if in_weights is not None:
        _check("moe_pairs.in_weights", in_weights, torch.float32)
    if (tuple(up.shape) != (E, F * (2 if gate_block else 1), W) or (in_weights is not None and in_weights.shape != weights.shape) or tuple(down.shape) != (E, W, F) or tuple(ids.shape) != (T, top)
            or tuple(weights.shape) != (T, top) or tuple(act_buf.shape) != (T * top, F) or tuple(out.shape) != (T, W)
            or (base is not None and tuple(base.shape) != (T, W))):
        raise KernelError(f"moe_pairs: h {tuple(h.shape)}, up {tuple(up.shape)}, down {tuple(down.shape)}, ids "
                          f"{tuple(ids.shape)}, activations {tuple(act_buf.shape)}, out {tuple(out.shape)}")
    code = library().q3_moe_pairs(h.data_ptr(), up.data_ptr(), down.data_ptr(), ids.data_ptr(), weights.data_ptr(),
                                  _ptr(base), act_buf.data_ptr(), out.data_ptr(), dtype_tag(h.dtype), T, W, F, E, top,
                                  activation_code(activation, gate=True), int(gate_block), _ptr(in_weights), _stream())
    _done("moe_pairs", code, f"experts {E}, top {top}, inner {F}")


MOE_GROUPED_FROM = 4  # tokens from which the sorted, grouped products run (below: a pair at a time)


def moe_tile_rows() -> int:
    """Rows per tile of the grouped products: every expert's rows start on a multiple of it."""
    if "moe tile rows" not in _DEVICE_FACTS:
        _DEVICE_FACTS["moe tile rows"] = int(library()._lib.q3_moe_tile_rows())
    return _DEVICE_FACTS["moe tile rows"]


def moe_grouped_tiles(num_tokens: int, top: int, experts: int) -> int:
    """The most tiles that the sorted rows of so many tokens can fill: every expert wastes less than one."""
    return (num_tokens * top) // moe_tile_rows() + experts


MOE_GATE_BLOCK = 16  # rows of a gated expert's stack alternate between gate and up in blocks of so many


def moe_gate_block(ff: int) -> int:
    """How the rows of a gated expert's two first matrices are interleaved: in blocks of ``MOE_GATE_BLOCK`` where the
    inner width is a multiple of it (the grouped product's epilogue then finds a gate and its up value in one piece),
    else all gate rows and then all up rows."""
    return MOE_GATE_BLOCK if ff % MOE_GATE_BLOCK == 0 else ff


def moe_grouped_takes(dtype: torch.dtype, width: int, ff: int, gated: bool = False) -> bool:
    """Whether the grouped products take these experts: bfloat16, rows of whole 16-byte pieces (gated experts: an
    inner width in multiples of ``MOE_GATE_BLOCK``)."""
    return dtype == torch.bfloat16 and width % 8 == 0 and ff % (MOE_GATE_BLOCK if gated else 8) == 0


class MoeScratch:
    """What the grouped products of at most ``max_tokens`` tokens keep between their kernels: the rows sorted by
    expert (input, activations, output), every pair's row, every row's pair, and the list of tiles."""

    def __init__(self, alloc, max_tokens: int, top: int, experts: int, width: int, ff: int):
        rows = moe_grouped_tiles(max_tokens, top, experts) * moe_tile_rows()
        self.sorted_in = alloc("moe.sorted_in", rows, width)
        self.sorted_act = alloc("moe.sorted_act", rows, ff)
        self.sorted_out = alloc("moe.sorted_out", rows, width)
        self.pos = alloc("moe.pos", max_tokens * top, dtype=torch.int32)
        self.src = alloc("moe.src", rows, dtype=torch.int32)
        self.meta = alloc("moe.meta", 1 + rows // moe_tile_rows(), dtype=torch.int32)


def moe_grouped(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                base: Optional[torch.Tensor], out: torch.Tensor, activation: str, scratch: MoeScratch,
                status: torch.Tensor, gated: bool = False, in_weights: Optional[torch.Tensor] = None) -> None:
    """out = base + sum_k weights[:, k] * down[ids[:, k]] act(up[ids[:, k]] h) for many tokens (bfloat16): the pairs
    sorted by expert into whole tiles, both products of all experts as one grouped tensor-core product each."""
    _check("moe_grouped.h", h, torch.bfloat16)
    _check("moe_grouped.up", up, torch.bfloat16)
    _check("moe_grouped.down", down, torch.bfloat16)
    _check("moe_grouped.ids", ids, torch.int32)
    _check("moe_grouped.weights", weights, torch.float32)
    _check("moe_grouped.out", out, torch.bfloat16)
    T, W = h.shape
    E, F = up.shape[0], up.shape[1] // (2 if gated else 1)
    top = ids.shape[1]
    if in_weights is not None:
        _check("moe_grouped.in_weights", in_weights, torch.float32)
    tiles = moe_grouped_tiles(T, top, E)
    rows = tiles * moe_tile_rows()
    if base is not None:
        _check("moe_grouped.base", base, torch.bfloat16)
    if (tuple(up.shape) != (E, F * (2 if gated else 1), W) or tuple(down.shape) != (E, W, F) or tuple(ids.shape) != (T, top)
            or (in_weights is not None and in_weights.shape != weights.shape)
            or tuple(weights.shape) != (T, top) or tuple(out.shape) != (T, W) or (base is not None and base.shape != h.shape)
            or scratch.sorted_in.shape[0] < rows or scratch.sorted_in.shape[1] != W or scratch.sorted_act.shape[1] != F
            or scratch.sorted_out.shape[1] != W or scratch.pos.numel() < T * top):
        raise KernelError(f"moe_grouped: h {tuple(h.shape)}, up {tuple(up.shape)}, down {tuple(down.shape)}, ids "
                          f"{tuple(ids.shape)}, out {tuple(out.shape)}, sorted rows {tuple(scratch.sorted_in.shape)}")
    # the tensor maps cover the whole of the scratch rows, so that every step's maps are the same few
    cap = scratch.sorted_in.shape[0] // moe_tile_rows()
    code = library().q3_moe_grouped(h.data_ptr(), up.data_ptr(), down.data_ptr(), ids.data_ptr(), weights.data_ptr(),
                                    _ptr(base), out.data_ptr(), scratch.sorted_in.data_ptr(), scratch.sorted_act.data_ptr(),
                                    scratch.sorted_out.data_ptr(), scratch.pos.data_ptr(), scratch.src.data_ptr(),
                                    scratch.meta.data_ptr(), T, W, F, E, top, cap, activation_code(activation, gate=True),
                                    1 if gated else 0, _ptr(in_weights), status.data_ptr(), _stream())
    _done("moe_grouped", code, f"experts {E}, top {top}, width {W}, ff {F}")


def routed_experts(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                   base: Optional[torch.Tensor], act_buf: torch.Tensor, out: torch.Tensor, activation: str,
                   scratch: Optional[MoeScratch] = None, status: Optional[torch.Tensor] = None, gate_block: int = 0,
                   in_weights: Optional[torch.Tensor] = None) -> None:
    """The chosen experts of a step's tokens, by the kernels that suit dtype and shape: with ``scratch``, from
    ``MOE_GROUPED_FROM`` tokens on, the grouped tensor-core products; otherwise a pair at a time (``moe_pairs``)."""
    if scratch is not None and status is not None and h.shape[0] >= MOE_GROUPED_FROM:
        moe_grouped(h, up, down, ids, weights, base, out, activation, scratch, status, gated=gate_block > 0,
                    in_weights=in_weights)
    else:
        moe_pairs(h, up, down, ids, weights, base, act_buf, out, activation, gate_block, in_weights)


# ------------------------------------------------------------------ Dynamic Tanh around sub-layers, a token's second embedding
def add_dyt(stream: torch.Tensor, delta: Optional[torch.Tensor], after, before, out: Optional[torch.Tensor],
            rows_add: Optional[torch.Tensor] = None, vec_add: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None) -> None:
    """stream += after(delta) + rows_add + vec_add (each optional), then out = before(stream).  ``after`` and ``before``
    are (alpha, weight, bias) of a Dynamic Tanh, tanh(alpha x) w + b, alpha a float32 tensor of one value on the
    device, or None for the identity.  ``out``: [T, W] in the compute dtype or float32, or None.  ``rows`` (int32):
    only these rows are worked out, into ``out`` [len(rows), W], and the stream stays as it is."""
    _check("add_dyt.stream", stream, torch.float32)
    T, W = stream.shape
    dtype = delta.dtype if delta is not None else (out.dtype if out is not None else torch.float32)
    if delta is not None:
        _check("add_dyt.delta", delta)
    if out is not None:
        _check("add_dyt.out", out)
        if out.dtype != dtype and out.dtype != torch.float32:
            raise KernelError(f"add_dyt: out is {out.dtype}, the step's dtype is {dtype}")
    for name, t in (("rows_add", rows_add), ("vec_add", vec_add)):
        if t is not None:
            _check(f"add_dyt.{name}", t, torch.float32)
    args = []
    for name, norm in (("after", after), ("before", before)):
        if norm is None:
            args += [None, None, None]
            continue
        alpha, weight, bias = norm
        for t in (alpha, weight, bias):
            _check(f"add_dyt.{name}", t, torch.float32)
        if alpha.numel() != 1 or weight.numel() != W or bias.numel() != W:
            raise KernelError(f"add_dyt: {name} has alpha {tuple(alpha.shape)}, weight {tuple(weight.shape)} for width {W}")
        args += [alpha.data_ptr(), weight.data_ptr(), bias.data_ptr()]
    R = 0
    if rows is not None:
        _check("add_dyt.rows", rows, torch.int32)
        R = rows.numel()
    n = R if rows is not None else T
    if ((delta is not None and tuple(delta.shape) != (T, W)) or (out is not None and tuple(out.shape) != (n, W))
            or (rows_add is not None and tuple(rows_add.shape) != (T, W)) or (vec_add is not None and vec_add.numel() != W)
            or (rows is not None and out is None)):
        raise KernelError(f"add_dyt: stream {tuple(stream.shape)}, delta {None if delta is None else tuple(delta.shape)}, "
                          f"out {None if out is None else tuple(out.shape)}")
    out_f32 = out is not None and out.dtype == torch.float32 and dtype != torch.float32
    code = library().q3_add_dyt(stream.data_ptr(), _ptr(delta), args[0], args[1], args[2], _ptr(rows_add), _ptr(vec_add),
                                args[3], args[4], args[5], _ptr(out), 1 if out_f32 else 0, _ptr(rows), R, dtype_tag(dtype),
                                T, W, _stream())
    _done("add_dyt", code, f"rows {n}, width {W}")


def side_gate(p: torch.Tensor, side: torch.Tensor, column: int, out: torch.Tensor) -> None:
    """out = gelu_tanh(p) * side[:, column : column + dim]; p, out [T, dim] in the compute dtype, side float32 [T, any]."""
    _check("side_gate.p", p)
    _check("side_gate.out", out, p.dtype)
    _check("side_gate.side", side, torch.float32)
    T, dim = p.shape
    if tuple(out.shape) != (T, dim) or side.shape[0] != T or column < 0 or column + dim > side.shape[1]:
        raise KernelError(f"side_gate: p {tuple(p.shape)}, side {tuple(side.shape)}, column {column}")
    code = library().q3_side_gate(p.data_ptr(), side.data_ptr(), side.shape[1], int(column), out.data_ptr(),
                                  dtype_tag(p.dtype), T, dim, _stream())
    _done("side_gate", code)


def add_unit_rms(stream: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """stream += y / sqrt(mean(y^2) + eps) * weight, row by row; stream float32 [T, W], y [T, W] in the compute dtype."""
    _check("add_unit_rms.stream", stream, torch.float32)
    _check("add_unit_rms.y", y)
    _check("add_unit_rms.weight", weight, torch.float32)
    T, W = stream.shape
    if tuple(y.shape) != (T, W) or weight.numel() != W:
        raise KernelError(f"add_unit_rms: stream {tuple(stream.shape)}, y {tuple(y.shape)}, weight {tuple(weight.shape)}")
    code = library().q3_add_unit_rms(stream.data_ptr(), y.data_ptr(), weight.data_ptr(), float(eps), dtype_tag(y.dtype), T,
                                     W, _stream())
    _done("add_unit_rms", code)


def sigmoid_gate(x: torch.Tensor, proj: torch.Tensor, column: int) -> None:
    """x *= sigmoid(proj[:, column : column + n]) in place, n = x.shape[1]; x may be a column view of a wider buffer."""
    if (x.dim() != 2 or x.stride(1) != 1 or not x.is_cuda or proj.dtype != x.dtype or proj.shape[0] != x.shape[0]
            or column < 0 or column + x.shape[1] > proj.shape[1]):
        raise KernelError(f"sigmoid_gate: x {tuple(x.shape)} strides {x.stride()}, proj {tuple(proj.shape)}, column {column}")
    _check("sigmoid_gate.proj", proj)
    code = library().q3_sigmoid_gate(x.data_ptr(), x.stride(0), proj.data_ptr(), proj.shape[1], int(column), x.shape[1],
                                     dtype_tag(x.dtype), x.shape[0], _stream())
    _done("sigmoid_gate", code)


# ------------------------------------------------------------------ the matrix memory of the xLSTM
def mlstm_max_dim() -> int:
    """The largest key size per head that ``mlstm_scan`` takes."""
    if "mlstm max dim" not in _DEVICE_FACTS:
        _DEVICE_FACTS["mlstm max dim"] = int(library()._lib.q3_mlstm_max_dim())
    return _DEVICE_FACTS["mlstm max dim"]


MLSTM_SEGMENT = 128       # tokens of a segment of the segmented scan
MLSTM_SEGMENTED_FROM = 256  # the longest portion of a step from which the segments can pay
# measured on a B200 (keys of 128, values of 256, 4 and 8 heads; keys of 32, values of 48): the single walk takes
# 0.43 us a token whatever the sizes (one warp per scheduler, bound by its own chain); the segmented form's two walks
# take 6.5e-7 us per token and value of the memory (bound by issue), and its list and carry some 30 us
MLSTM_WALK_US_PER_TOKEN = 0.43
MLSTM_SEGMENTS_US_PER_TOKEN_VALUE = 6.5e-7
MLSTM_SEGMENTS_FIXED_US = 30.0


def mlstm_segmented_pays(dtype: torch.dtype, max_q_len: int, num_tokens: Optional[int] = None,
                         memory_values: Optional[int] = None) -> bool:
    """Whether a step runs the scan in segments side by side: bfloat16 (the float32 run keeps the single walk, whose sums
    have one order whatever the cut), a portion long enough to be cut, and (given the step's tokens and heads * dim * vdim)
    the walk of the longest portion slower than both walks of all tokens: several long portions already run side by
    side in the single walk."""
    if dtype != torch.bfloat16 or max_q_len < MLSTM_SEGMENTED_FROM:
        return False
    if num_tokens is None or memory_values is None:
        return True
    return (MLSTM_WALK_US_PER_TOKEN * max_q_len
            > MLSTM_SEGMENTS_FIXED_US + MLSTM_SEGMENTS_US_PER_TOKEN_VALUE * num_tokens * memory_values)


class MlstmScratch:
    """What the segmented scan of at most ``max_tokens`` tokens of ``max_seqs`` requests keeps between its kernels."""

    def __init__(self, alloc, max_tokens: int, max_seqs: int, heads: int, dim: int, vdim: int):
        self.max_segments = max_tokens // MLSTM_SEGMENT + max_seqs
        n = self.max_segments
        self.segments = alloc("mlstm.segments", n * 4, dtype=torch.int32)
        self.first_of = alloc("mlstm.first_of", max_seqs + 1, dtype=torch.int32)
        self.memory = alloc("mlstm.seg_memory", n * heads * vdim * dim, dtype=torch.float32)
        self.normaliser = alloc("mlstm.seg_normaliser", n * heads * dim, dtype=torch.float32)
        self.maxima = alloc("mlstm.seg_maxima", 3 * n * heads, dtype=torch.float32)


def mlstm_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, i_col: int, f_col: int, i_bias: torch.Tensor,
               f_bias: torch.Tensor, cap: float, memory: torch.Tensor, normaliser: torch.Tensor, maximum: torch.Tensor,
               q_start: torch.Tensor, slot_ids: torch.Tensor, num_seqs: int, out: torch.Tensor, status: torch.Tensor,
               max_q_len: int = 1, scratch: Optional[MlstmScratch] = None) -> None:
    """The mLSTM recurrence over every request's tokens in order.  ``proj`` [T, any]: q and k (heads * dim each), v
    (heads * vdim) and the two gates' pre-activations (heads each) from the given columns; state per slot: ``memory``
    [slots, heads, vdim, dim] (the memory column by column), ``normaliser`` [slots, heads, dim], ``maximum`` [slots, heads], float32, read and
    renewed; ``out`` float32 [T, heads * vdim]: S^T q / (max(|n . q|, exp(-m)) + 1e-6) with q times dim^-1/2.  With
    ``scratch`` and a step for which ``mlstm_segmented_pays``, every portion is cut into segments that are walked side
    by side (each from an empty memory, then a carry through a request's segments, then the walk that writes)."""
    _check("mlstm_scan.proj", proj)
    for name, t in (("i_bias", i_bias), ("f_bias", f_bias), ("memory", memory), ("normaliser", normaliser),
                    ("maximum", maximum), ("out", out)):
        _check(f"mlstm_scan.{name}", t, torch.float32)
    for name, t in (("q_start", q_start), ("slot_ids", slot_ids)):
        _check(f"mlstm_scan.{name}", t, torch.int32)
    T, ld = proj.shape
    slots, H, Dv, D = memory.shape
    if (tuple(normaliser.shape) != (slots, H, D) or tuple(maximum.shape) != (slots, H) or tuple(out.shape) != (T, H * Dv)
            or i_bias.numel() != H or f_bias.numel() != H or min(q_col, k_col, v_col, i_col, f_col) < 0
            or max(q_col + H * D, k_col + H * D, v_col + H * Dv, i_col + H, f_col + H) > ld):
        raise KernelError(f"mlstm_scan: proj {tuple(proj.shape)}, memory {tuple(memory.shape)}, out {tuple(out.shape)}")
    seg, max_segments, extra = 0, 0, [None] * 5
    if scratch is not None and mlstm_segmented_pays(proj.dtype, max_q_len, T, H * D * Dv):
        seg, max_segments = MLSTM_SEGMENT, T // MLSTM_SEGMENT + int(num_seqs)
        if (max_segments > scratch.max_segments or scratch.memory.numel() < max_segments * H * Dv * D
                or scratch.first_of.numel() < num_seqs + 1):
            raise KernelError(f"mlstm_scan: the scratch holds {scratch.max_segments} segments, the step needs {max_segments}")
        extra = [scratch.segments.data_ptr(), scratch.first_of.data_ptr(), scratch.memory.data_ptr(),
                 scratch.normaliser.data_ptr(), scratch.maxima.data_ptr()]
    code = library().q3_mlstm_scan(proj.data_ptr(), ld, int(q_col), int(k_col), int(v_col), int(i_col), int(f_col),
                                   i_bias.data_ptr(), f_bias.data_ptr(), float(cap), memory.data_ptr(),
                                   normaliser.data_ptr(), maximum.data_ptr(), q_start.data_ptr(), slot_ids.data_ptr(),
                                   slots, out.data_ptr(), dtype_tag(proj.dtype), int(num_seqs), H, D, Dv, seg, max_segments,
                                   *extra, status.data_ptr(), _stream())
    _done("mlstm_scan", code, f"heads {H}, dim {D}, vdim {Dv}")


def mlstm_out(o: torch.Tensor, proj: torch.Tensor, g_col: int, weight: torch.Tensor, eps: float, out: torch.Tensor,
              out_scale: float, heads: int) -> None:
    """out = o / rms_per_head(o) * weight * sigmoid(proj[:, g_col:]) * out_scale; o float32 [T, heads * vdim]; ``out`` in
    the compute dtype, possibly a column view of a wider buffer."""
    _check("mlstm_out.o", o, torch.float32)
    _check("mlstm_out.proj", proj)
    _check("mlstm_out.weight", weight, torch.float32)
    T, n = o.shape
    if (n % heads or out.dtype != proj.dtype or out.dim() != 2 or tuple(out.shape) != (T, n) or out.stride(1) != 1
            or weight.numel() != n or g_col < 0 or g_col + n > proj.shape[1] or proj.shape[0] != T):
        raise KernelError(f"mlstm_out: o {tuple(o.shape)}, proj {tuple(proj.shape)}, out {tuple(out.shape)}")
    code = library().q3_mlstm_out(o.data_ptr(), proj.data_ptr(), proj.shape[1], int(g_col), weight.data_ptr(), float(eps),
                                  float(out_scale), out.data_ptr(), out.stride(0), dtype_tag(proj.dtype), T, int(heads),
                                  n // heads, _stream())
    _done("mlstm_out", code)
