"""The kernels of the step, as Python calls on torch tensors.

``get_ops(device)`` loads the compiled sm_100a library (building it first if it is missing
or stale) and returns the one ``CudaOps`` object every part calls.  There is no other
implementation behind these calls: without a CUDA device or without the library they raise.
Every call launches on torch's current stream of the tensors' device and returns at once.

Matrix products of the bfloat16 path go to the library product (cuBLAS through
``torch.mm``), as the reference's ``nn.Linear`` layers do (models/mqa.py:123-126,
models/mlp.py:20-22); the float32 path uses this package's own FFMA kernel so that no
reduced-precision matrix mode can slip in.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from . import build as _build

_DT = {torch.float32: 0, torch.bfloat16: 1}
_c_int, _c_ll, _c_float, _c_void = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p

_SIGNATURES = {
    "ttie_embed": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ttie_add_rmsnorm": [_c_void, _c_void, _c_void, _c_int, _c_ll, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int,
                         _c_float, _c_int, _c_void],
    "ttie_rope_store_partial": [_c_void, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_int,
                                _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_rope_table": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_void],
    "ttie_rope_table_scaled": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_float, _c_void],
    "ttie_rope_store_vec": [_c_void, _c_ll, _c_void, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void,
                            _c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_skinny_gemm": [_c_void, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_void],
    "ttie_skinny_gemm_tuned": [_c_void, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int,
                               _c_int, _c_int, _c_void],
    "ttie_swiglu": [_c_void, _c_void, _c_int, _c_int, _c_int, _c_void],
    "ttie_rope_store": [_c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_int, _c_void,
                        _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_gemm_f32": [_c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_paged_attention": [_c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_int, _c_int,
                             _c_void, _c_int, _c_void],
    "ttie_paged_attention_mma": [_c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                                 _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_int, _c_int,
                                 _c_void, _c_void],
    "ttie_paged_attention_mma_form": [_c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                                      _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_int, _c_int,
                                      _c_void, _c_int, _c_void],
    "ttie_paged_attention_weights": [_c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_int, _c_int,
                                     _c_void, _c_int, _c_int, _c_void, _c_void],
    "ttie_paged_attention_mma_weights": [_c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                                         _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_int, _c_int,
                                         _c_void, _c_int, _c_int, _c_void, _c_void],
    "ttie_paged_attention_tc": [_c_void, _c_ll, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                                _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int,
                                _c_void],
    "ttie_paged_attention_tc_weights": [_c_void, _c_ll, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_void, _c_void, _c_void,
                                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int,
                                        _c_int, _c_void, _c_void],
    "ttie_gemm_tc": [_c_void, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_gemm_tc_pair": [_c_void, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_scale_add_layernorm": [_c_void, _c_void, _c_int, _c_void, _c_int, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int,
                                 _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_void],
    "ttie_cast_rows": [_c_void, _c_void, _c_ll, _c_int, _c_void],
    "ttie_latent_store": [_c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int, _c_float, _c_void, _c_void, _c_void,
                          _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_latent_query": [_c_void, _c_ll, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void],
    "ttie_gate_heads": [_c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int, _c_void],
    "ttie_rmsnorm_cols": [_c_void, _c_ll, _c_int, _c_int, _c_int, _c_void, _c_int, _c_float, _c_void, _c_int, _c_void],
    "ttie_gemm_f32_batched": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll, _c_ll, _c_ll, _c_void],
    "ttie_causal_conv": [_c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int, _c_void, _c_void,
                         _c_void, _c_void, _c_void, _c_int, _c_void],
    "ttie_rglru_scan": [_c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_void, _c_ll, _c_int, _c_void, _c_ll, _c_int, _c_void,
                        _c_int, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void, _c_int, _c_void,
                        _c_int, _c_void],
    "ttie_glu": [_c_void, _c_ll, _c_void, _c_int, _c_int, _c_float, _c_float, _c_float, _c_int, _c_void],
    "ttie_moe_route": [_c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void],
    "ttie_moe_plan": [_c_void, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void],
    "ttie_grouped_gemm": [_c_void, _c_ll, _c_void, _c_int, _c_void, _c_ll, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_int, _c_int, _c_int,
                          _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_float, _c_void],
    "ttie_grouped_gemm_act": [_c_void, _c_ll, _c_void, _c_int, _c_void, _c_ll, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_int, _c_int, _c_int,
                              _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_float, _c_int, _c_void, _c_void, _c_void],
    "ttie_row_scale_act": [_c_void, _c_ll, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void],
    "ttie_moe_combine_gated": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int, _c_void, _c_ll,
                               _c_void, _c_ll, _c_void],
    "ttie_skinny_gemm_glu": [_c_void, _c_ll, _c_void, _c_ll, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_float, _c_float, _c_float, _c_void],
    "ttie_gather_rows": [_c_void, _c_ll, _c_void, _c_int, _c_int, _c_int, _c_void, _c_int, _c_void],
    "ttie_moe_combine": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int, _c_void, _c_ll, _c_void],
    "ttie_qkv_conv_rope_store": [_c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void,
                                 _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_float, _c_void, _c_int, _c_float, _c_int,
                                 _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
    "ttie_proj_row_rms": [_c_void, _c_ll, _c_int, _c_int, _c_int, _c_float, _c_void, _c_int, _c_void],
    "ttie_stream_conv": [_c_void, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void],
    "ttie_conv_tail_update": [_c_void, _c_ll, _c_int, _c_int, _c_void, _c_int, _c_void, _c_void, _c_int, _c_int, _c_void],
    "ttie_gate_head_rows": [_c_void, _c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int, _c_void],
    "ttie_token_shift_mix": [_c_void, _c_ll, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int,
                             _c_void],
    "ttie_wkv_decay": [_c_void, _c_ll, _c_void, _c_void, _c_int, _c_int, _c_void],
    "ttie_wkv_scan": [_c_void, _c_void, _c_void, _c_ll, _c_void, _c_void, _c_void, _c_int, _c_void, _c_ll, _c_int, _c_void,
                      _c_int, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_void],
    "ttie_mlstm_gates": [_c_void, _c_ll, _c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int, _c_float, _c_void, _c_void, _c_int,
                         _c_void],
    "ttie_mlstm_scan": [_c_void, _c_void, _c_void, _c_ll, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_void, _c_int,
                        _c_void, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void],
    "ttie_rotate_heads": [_c_void, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int, _c_float, _c_void, _c_int, _c_void],
    "ttie_retention_scan": [_c_void, _c_void, _c_ll, _c_void, _c_ll, _c_void, _c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int,
                            _c_int, _c_int, _c_int, _c_void, _c_int, _c_void],
    "ttie_head_norm_gate": [_c_void, _c_void, _c_ll, _c_void, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void, _c_int, _c_void],
    "ttie_activation": [_c_void, _c_void, _c_ll, _c_int, _c_float, _c_int, _c_int, _c_void],
    "ttie_matrix_state_pad": [_c_int],
    "ttie_sample": [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void],
    "ttie_sample_tuned": [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void],
}


class KernelError(RuntimeError):
    pass


def _row_bucket(M: int) -> int:
    return 16 if M <= 16 else 32 if M <= 32 else 64


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class CudaOps:
    name = "cuda-sm100a"

    def __init__(self, device):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine computes only with its sm_100a kernels "
                              "(there is no CPU path)")
        self.device = torch.device(device)
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"the kernel library is built for sm_100a (B200); device reports sm_{major}{minor}")
        path = _build.build()
        self.lib_path = path
        self.lib = ctypes.CDLL(path)
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = argtypes, _c_int
        self.lib.ttie_last_error.restype = ctypes.c_char_p
        self.launches = 0                     # kernels of this library launched so far
        self.num_sms = int(torch.cuda.get_device_properties(self.device).multi_processor_count)   # the plans below are sized for it
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or \
            (lambda index: torch.cuda.current_stream(index).cuda_stream)
        self.attn_target_ctas = 4 * self.num_sms  # decode tiles are small: four CTAs share an SM
        self.attn_cluster_max_rows = 64         # query rows per request (tokens x heads per kv head) up to which the decode form runs
        self.attn_cluster_max_size = 8          # CTAs per cluster (16 is placed on fewer SMs at a time)
        self.attn_cluster_tiles_per_warp = 1    # ... and only while a warp walks at most this many 64-key tiles
        self._cluster_max = {}
        self._mma_per_sm = {}
        self._plans = {}
        self.attn_tc_min_rows = 256             # query rows per request from which the tcgen05 attention kernel is used
        self.skinny_max_rows = 8                # rows up to which the weight-streaming product is the rule (tune_products may hand a shape to the library)
        self._swiglu_choice = {}                # (F, K, row bucket) -> True where the fused tcgen05 gate/up + SwiGLU kernel measured faster
        self._product_choice = {}               # (N, K, row bucket[, "split"]) -> "skinny" | "library" (tune_products; "split": for callers that take partial sums)
        self._skinny_tuned = {}                 # (N, K, row bucket 8 | 16) -> (K range per CTA, form code) where tune_products found a faster form
        self._grouped_mm = None                 # the library's grouped product: None = not looked up yet, False = this build has none
        self.product_timings = {}               # what tune_products measured: (N, K, rows) -> {"library": ms, "skinny": ms (best form), "skinny_uncut": ms, ...}
        self.lib.ttie_attn_tc_supported.restype = _c_int
        if os.environ.get("TTIE_NVTX", "0") not in ("", "0"):
            self._wrap_in_ranges()
        self._tc_pinned = torch.zeros(2, dtype=torch.int32).pin_memory()       # failure codes of the tcgen05 kernels, written by the device
        self._tc_words = self._tc_pinned.numpy()
        for i, name in enumerate(("ttie_gemm_tc_set_mirror", "ttie_attn_tc_set_mirror")):
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = [_c_void], _c_int
            if fn(self._tc_pinned.data_ptr() + 4 * i):
                raise KernelError(f"{name} failed")
        for name in ("ttie_attn_mma_supported", "ttie_attn_mma_tile_rows", "ttie_attn_cluster_tile_rows", "ttie_attn_cluster_active",
                     "ttie_attn_mma_ctas_per_sm"):
            getattr(self.lib, name).restype = _c_int

    # ------------------------------------------------------------------ helpers
    _RANGED = ("embed", "add_rmsnorm", "rmsnorm_rows", "linear", "linear_swiglu", "swiglu", "rope_table", "rope_store",
               "paged_attention", "sample")

    def _wrap_in_ranges(self):
        """With ``TTIE_NVTX=1`` in the environment every operation below opens an NVTX range of its own name around its
        launches, so a timeline of a step reads op by op (the reference marks the same places with
        ``torch.profiler.record_function`` behind its ``PROFILE_REGIONS`` flag, models/mqa.py:14-18).  Off by
        default: the step's host time is too short to spend on it unasked."""
        push, pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop

        def ranged(name, fn):
            def call(*args, **kwargs):
                push(name)
                try:
                    return fn(*args, **kwargs)
                finally:
                    pop()
            return call

        for name in self._RANGED:
            setattr(self, name, ranged(name, getattr(self, name)))

    def _check(self, rc: int, what: str):
        if rc != 0:
            raise KernelError(f"{what}: {self.lib.ttie_last_error().decode()}")

    def _stream(self, t: torch.Tensor = None):
        """torch's current stream of the device as a raw handle (asked at every call: a graph capture changes it).
        The direct query is an order of magnitude cheaper than building a ``torch.cuda.Stream`` object, which
        counts on steps that are not replayed from a graph."""
        return self._raw_stream(self._device_index)

    @staticmethod
    def _dt(t: torch.Tensor) -> int:
        try:
            return _DT[t.dtype]
        except KeyError:
            raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None

    # ------------------------------------------------------------------ what the kernels take
    def check_dtype(self, dtype):
        if dtype not in _DT:
            raise KernelError(f"dtype {dtype} is not supported (float32 or bfloat16)")

    def check_attention(self, dtype, num_heads, num_kv_heads, head_dim, page_size):
        """Raises unless some attention kernel here takes the sizes: the general kernel takes every head size that is
        a multiple of 4 up to 512, any head counts and any page size (the tensor-core kernels cover subsets of that)."""
        self.check_dtype(dtype)
        if head_dim <= 0 or head_dim % 4 or head_dim > 512:
            raise KernelError(f"attention: head size {head_dim} not supported (multiples of 4 up to 512)")
        if num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise KernelError(f"attention: {num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        if page_size < 1:
            raise KernelError(f"attention: page size {page_size}")

    def check_norm(self, dtype, dim):
        self.check_dtype(dtype)
        if dim * 4 > 200 * 1024:
            raise KernelError(f"rmsnorm: width {dim} needs {dim * 4} bytes of shared memory (limit 204800)")

    # ------------------------------------------------------------------ ops
    def embed(self, token_ids, table, out, scale=1.0):
        """out[t] = table[token_ids[t]] * scale (float32)."""
        T, d = out.shape
        self._check(self.lib.ttie_embed(_ptr(token_ids), _ptr(table), _ptr(out), T, d, table.shape[0], float(scale),
                                        self._dt(table), self._stream(out)), "embed")
        self.launches += 1

    @staticmethod
    def _delta_args(delta):
        """(delta pointer, partial pointer, S, stride) for a delta that is None, [T, d] in the compute
        dtype, float32 [T, d], or float32 partial sums [S, T, d]."""
        if delta is None:
            return None, None, 0, 0
        if delta.dim() == 3:
            return None, delta.data_ptr(), delta.shape[0], delta.stride(0)
        if delta.dtype == torch.float32:                     # one 32-bit sum [T, d], whatever the compute dtype
            return None, delta.data_ptr(), 1, 0
        return delta.data_ptr(), None, 0, 0

    def add_rmsnorm(self, resid, delta, weight, eps, out):
        R, d = resid.shape
        dp, pp, S, stride = self._delta_args(delta)
        self._check(self.lib.ttie_add_rmsnorm(_ptr(resid), dp, pp, S, stride, None, _ptr(weight), self._dt(weight),
                                              _ptr(out), R, d, float(eps), self._dt(out), self._stream(out)), "add_rmsnorm")
        self.launches += 1

    def rmsnorm_rows(self, resid, delta, rows, num_rows, weight, eps, out):
        d = resid.shape[1]
        dp, pp, S, stride = self._delta_args(delta)
        self._check(self.lib.ttie_add_rmsnorm(_ptr(resid), dp, pp, S, stride, _ptr(rows), _ptr(weight), self._dt(weight),
                                              _ptr(out), num_rows, d, float(eps), self._dt(out), self._stream(out)),
                    "rmsnorm_rows")
        self.launches += 1

    # ---- matrix products
    def _skinny_ok(self, x, w, may_split=False):
        """Whether the weight-streaming product takes this product.  ``may_split``: the caller accepts partial sums of a
        K range cut over CTAs; the measured choice for such calls (which may rest on a cut form) is kept apart."""
        M = x.shape[0]
        key = (w.shape[0], w.shape[1], 8 if M <= self.skinny_max_rows else _row_bucket(M)) + (("split",) if may_split else ())
        choice = self._product_choice.get(key)
        if M > self.skinny_max_rows and not (M <= 64 and choice == "skinny"):
            return False
        if M <= self.skinny_max_rows and choice == "library":
            return False
        return (x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
                and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)

    def tune_products(self, weights, iters=8):
        """Which product serves each distinct bfloat16 matrix shape of a model at 8, 16, 32 and 64 rows, by measurement:
        a replayed graph of ``iters`` launches that rotate over the model's matrices of that shape (so that the weights come
        from HBM).  For 9 to 64 rows neither this package's weight-streaming product nor the library's wins at every
        shape (at the Llama-2-7B widths the library is ahead by 10-20 % from 32 rows on; on a narrow, deep matrix such as
        [2048, 16384] it leaves half of the memory bandwidth unused), and the faster one is remembered.  Up to 8 rows the
        weight-streaming product is the rule and is ahead on most shapes, by up to 3x on narrow deep ones; a shape goes to
        the library where that is more than 5 % faster (measured: [10240, 8192] and [8192, 28672] by 9-10 %).  At 8 and
        16 rows the weight-streaming product's own form is measured too - K cut into 1 to 16 ranges over CTAs, one or two
        sets of 16 weight rows per CTA - and a form that beats the rule of thumb (``_kslice``) by 3 % is kept: [4352, 4096]
        at 8 rows takes 7.8 us in 6 ranges with two row sets against 9.1 in 8 ranges with one, [4544, 18176] 28.5 us in 6
        ranges against 38.3 uncut.  Small matrices (under 4 Mi elements) are left alone."""
        groups, launches = {}, self.launches
        for w in weights:
            if w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1 and w.shape[0] * w.shape[1] >= (4 << 20):
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        for (N, K), ws in groups.items():
            for M in (8, 16, 32, 64):
                if (N, K, M) in self._product_choice:
                    continue
                x = torch.randn(M, K, device=self.device).to(torch.bfloat16)
                if not self._skinny_shape_ok(x, ws[0]):
                    continue

                def measure(kind, form=None, partial_ok=True):
                    self._product_choice[(N, K, M)] = self._product_choice[(N, K, M, "split")] = kind
                    self._skinny_tuned.pop((N, K, M), None)
                    if form is not None:
                        self._skinny_tuned[(N, K, M)] = form
                    return self._graph_time_rotating(lambda i: self.linear(x, ws[i % len(ws)], None, partial_ok=partial_ok), iters)

                def decide(skinny, library):
                    if M == 8:  # up to 8 rows the weight-streaming product is the rule; the library takes a shape only where it is clearly ahead
                        return "library" if library < 0.95 * skinny else "skinny"
                    return "skinny" if skinny < 0.97 * library else "library"

                took = {"library": measure("library"), "skinny_uncut": measure("skinny", partial_ok=False), "skinny": measure("skinny")}
                form = None
                if M <= 16:
                    # up to 16 rows the weight-streaming product's own form is measured as well: one or two sets of 16 weight
                    # rows per CTA, K cut into 1 to 16 ranges
                    for code in (0, 16):
                        for S in (1, 2, 3, 4, 6, 8, 12, 16):
                            kslice = math.ceil(math.ceil(K / S) / 128) * 128
                            if kslice < 256 or math.ceil(K / kslice) != S:
                                continue
                            t = measure("skinny", (kslice, code))
                            if t < 0.97 * took["skinny"]:
                                took["skinny"], form = t, (kslice, code)
                self._skinny_tuned.pop((N, K, M), None)
                if form is not None:
                    self._skinny_tuned[(N, K, M)] = form
                    took["skinny_form"] = {"k_ranges": math.ceil(K / form[0]), "row_sets": 2 if form[1] & 16 else 1}
                # callers that take partial sums of a cut K range, and callers that want the whole sum
                self._product_choice[(N, K, M, "split")] = decide(took["skinny"], took["library"])
                self._product_choice[(N, K, M)] = decide(took["skinny_uncut"], took["library"])
                self.product_timings[(N, K, M)] = took
        self.launches = launches

    @staticmethod
    def _skinny_shape_ok(x, w):
        return x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0

    def _kslice(self, N, K, may_split):
        """K range per CTA of the weight-streaming kernel.  K is split over CTAs (partial sums) when the
        16-row tiles alone are too few to balance the SMs."""
        tiles = math.ceil(N / 16)
        full = math.ceil(K / 128) * 128
        if not may_split or tiles >= 4 * self.num_sms:
            return full
        best, best_eff = full, 0.0
        for S in (1, 2, 3, 4, 6, 8):
            ks = math.ceil(math.ceil(K / S) / 128) * 128
            if ks < 256:
                break
            ctas = tiles * math.ceil(K / ks)
            eff = (ctas / self.num_sms) / math.ceil(ctas / self.num_sms)
            if eff > best_eff + 0.02:
                best, best_eff = ks, eff
        return best

    def linear(self, x, w, bias, out_dtype=None, partial_ok=False):
        """y = x @ w.T (+ bias); x [M, K], w [N, K] -> [M, N].  With ``partial_ok`` the result may
        instead be float32 partial sums [S, M, N] of a K-split product, which ``add_rmsnorm``,
        ``rmsnorm_rows`` and ``rope_store`` accept and add up."""
        M, K = x.shape
        N = w.shape[0]
        if x.dtype == torch.float32:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
            self._check(self.lib.ttie_gemm_f32(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K, x.stride(0),
                                               w.stride(0), N, self._stream(x)), "gemm_f32")
            self.launches += 1
            return out
        may_split = partial_ok and bias is None and out_dtype is None
        if self._skinny_ok(x, w, may_split):
            tuned = self._skinny_tuned.get((N, K, 8 if M <= 8 else 16)) if (may_split and M <= 16) else None
            kslice, form = tuned if tuned is not None else (self._kslice(N, K, may_split), 0)
            S = math.ceil(K / kslice)
            if S > 1:
                out, epi = torch.empty((S, M, N), dtype=torch.float32, device=x.device), 1
            elif out_dtype == torch.float32:
                out, epi = torch.empty((M, N), dtype=torch.float32, device=x.device), 3
            else:
                out, epi = torch.empty((M, N), dtype=torch.bfloat16, device=x.device), 0
            self._check(self.lib.ttie_skinny_gemm_tuned(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out), N,
                                                        M, N, K, kslice, epi, 0, form, self._stream(x)), "skinny_gemm")
            self.launches += 1
            return out
        # bfloat16, many rows: the library product, 32-bit accumulation inside
        if out_dtype == torch.float32:
            out = torch.mm(x, w.t(), out_dtype=torch.float32)
            if bias is not None:
                out += bias.float()
            return out
        if bias is not None:
            return torch.addmm(bias, x, w.t())
        return torch.mm(x, w.t())

    def linear_tc(self, x, w, bias, out_dtype=None, tile_n=256):
        """The tcgen05 / TMA / TMEM product: y = x @ w.T (+ bias) for bfloat16 operands."""
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
        self._check(self.lib.ttie_gemm_tc(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out), out.stride(0),
                                          M, N, K, 1 if out.dtype == torch.float32 else 0, tile_n, self._stream(x)), "gemm_tc")
        self.launches += 1
        return out

    def linear_tc_pair(self, x, w, bias, out_dtype=None):
        """The tcgen05 product on pairs of CTAs (256 x 256 tiles): y = x @ w.T (+ bias) for bfloat16 operands."""
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
        self._check(self.lib.ttie_gemm_tc_pair(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out), out.stride(0),
                                               M, N, K, 1 if out.dtype == torch.float32 else 0, 0, self._stream(x)), "gemm_tc_pair")
        self.launches += 1
        return out

    def linear_swiglu_tc_pair(self, x, w_gu, b_gu, hidden):
        """silu(x @ Wg.T) * (x @ Wu.T) in one kernel: the pair product with the activation in its epilogue."""
        M, K = x.shape
        act = torch.empty((M, hidden), dtype=torch.bfloat16, device=x.device)
        self._check(self.lib.ttie_gemm_tc_pair(_ptr(x), x.stride(0), _ptr(w_gu), w_gu.stride(0), _ptr(b_gu), _ptr(act), act.stride(0),
                                               M, hidden, K, 0, 1, self._stream(x)), "gemm_tc_pair (SwiGLU)")
        self.launches += 1
        return act

    def tc_error(self) -> int:
        """Error word of the tcgen05 kernels (0 = none; otherwise the code of the first bounded wait that
        ran out: product 1-4, attention 101-110); synchronises the device."""
        g = int(self.lib.ttie_tc_error())
        a = int(self.lib.ttie_attn_tc_error())
        return g or (100 + a if a else 0)

    def check_tc(self):
        """After a point where the host has waited for the device: raises if a bounded wait inside a tcgen05
        kernel ran out since the last check (its result is then not to be trusted).  The kernels also write
        their failure code into two words of pinned host memory, so this costs two loads - it is called
        after every step, graph replays included."""
        if self._tc_words[0] or self._tc_words[1]:
            self._tc_words[:] = 0
            code = self.tc_error() or -1
            raise KernelError(f"a tcgen05 kernel gave up waiting on a barrier (code {code}); its output is invalid")

    def linear_swiglu(self, x, w_gu, b_gu, hidden):
        """silu(x @ Wg.T) * (x @ Wu.T) with w_gu = [Wg; Wu] ([2*hidden, K]) -> [M, hidden]."""
        M, K = x.shape
        act = torch.empty((M, hidden), dtype=x.dtype, device=x.device)
        if self._skinny_ok(x, w_gu) and self._fused_few_rows_wins(x, w_gu, b_gu, hidden):
            return self._linear_swiglu_skinny(x, w_gu, b_gu, hidden, act)
        if M >= 1024 and x.dtype == torch.bfloat16 and self._skinny_shape_ok(x, w_gu) and self._fused_swiglu_wins(x, w_gu, b_gu, hidden):
            return self.linear_swiglu_tc_pair(x, w_gu, b_gu, hidden)
        self.swiglu(self.linear(x, w_gu, b_gu), act)
        return act

    def _linear_swiglu_skinny(self, x, w_gu, b_gu, hidden, act):
        M, K = x.shape
        self._check(self.lib.ttie_skinny_gemm(_ptr(x), x.stride(0), _ptr(w_gu), w_gu.stride(0), _ptr(b_gu), _ptr(act),
                                              hidden, M, hidden, K, math.ceil(K / 128) * 128, 2, hidden,
                                              self._stream(x)), "skinny_gemm_swiglu")
        self.launches += 1
        return act

    def _graph_time_rotating(self, fn, iters=8) -> float:
        """Milliseconds of one replay of a graph of ``iters`` calls ``fn(i)`` (after two plain calls)."""
        for i in range(2):
            fn(i)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
        g.replay()
        best = None
        for _ in range(3):                                           # the least of three replays
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize(self.device)
            best = a.elapsed_time(b) if best is None else min(best, a.elapsed_time(b))
        return best

    def _graph_time(self, fn, iters=8) -> float:
        """Milliseconds of one replay of a graph of ``iters`` calls of ``fn`` (after two plain calls)."""
        for _ in range(2):
            fn()
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize(self.device)
        return a.elapsed_time(b)

    def _fused_few_rows_wins(self, x, w_gu, b_gu, hidden) -> bool:
        """Up to 8 rows: whether the weight-streaming product with SwiGLU in its epilogue beats the same product without
        it followed by the activation kernel.  The fused form cannot cut K over CTAs (the activation needs whole sums),
        so it has hidden / 16 CTAs: at the Llama-2-7B widths (688 CTAs) it is 8 % ahead, at a feed-forward width of
        2,048 to 4,096 behind a model width of 4,096 to 8,192 it is 15-40 % behind.  Measured per shape the first time
        it is met outside a graph capture (a step that meets a new batch bucket runs plainly once before it is
        captured), as a replayed graph of eight launches each."""
        key = (hidden, x.shape[1], "few")
        choice = self._swiglu_choice.get(key)
        if choice is None:
            if torch.cuda.is_current_stream_capturing():
                return True
            launches = self.launches
            act = torch.empty((x.shape[0], hidden), dtype=x.dtype, device=x.device)
            took = {"fused": self._graph_time(lambda: self._linear_swiglu_skinny(x, w_gu, b_gu, hidden, act)),
                    "unfused": self._graph_time(lambda: self.swiglu(self.linear(x, w_gu, b_gu), act))}
            self.launches = launches
            choice = self._swiglu_choice[key] = took["fused"] <= 1.03 * took["unfused"]
            self.product_timings[("swiglu",) + key] = took
        return choice

    def _fused_swiglu_wins(self, x, w_gu, b_gu, hidden) -> bool:
        """Whether, for portions of this many rows, the gate/up product with SwiGLU in its epilogue (this package's
        tcgen05 kernel on CTA pairs) is faster than the library's product followed by the activation kernel.  Measured
        the first time a shape and row bucket (1,024 / 2,048 / 4,096 rows and up) is met outside a graph capture: three
        launches of each between events.  At the Llama-2-7B and Falcon-7B widths the two are within 3 % of each other
        at 2,048 rows; below 1,024 rows the pair kernel has too few tiles for the GPU and is not considered."""
        M, K = x.shape
        key = (hidden, K, 4096 if M >= 4096 else 2048 if M >= 2048 else 1024)
        choice = self._swiglu_choice.get(key)
        if choice is None:
            if torch.cuda.is_current_stream_capturing():
                return False
            launches, took = self.launches, {}
            act = torch.empty((M, hidden), dtype=x.dtype, device=x.device)
            for kind, fn in (("library", lambda: self.swiglu(self.linear(x, w_gu, b_gu), act)),
                             ("pair", lambda: self.linear_swiglu_tc_pair(x, w_gu, b_gu, hidden))):
                fn()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(3):
                    fn()
                b.record()
                b.synchronize()
                took[kind] = a.elapsed_time(b)
            self.launches = launches
            choice = self._swiglu_choice[key] = took["pair"] < took["library"]
            self.product_timings[("swiglu",) + key] = took
        return choice

    def swiglu(self, gate_up, out):
        T, F = out.shape
        self._check(self.lib.ttie_swiglu(_ptr(gate_up), _ptr(out), T, F, self._dt(out), self._stream(out)), "swiglu")
        self.launches += 1

    def rope_table(self, positions, inv_freq, magnitude=1.0):
        """cos and sin of pos * inv_freq for every token of the step, both times ``magnitude``: float32 [T, D/2, 2]."""
        T, half = positions.shape[0], inv_freq.shape[0]
        cs = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
        self._check(self.lib.ttie_rope_table_scaled(_ptr(positions), _ptr(inv_freq), _ptr(cs), T, half, float(magnitude), self._stream(cs)),
                    "rope_table")
        self.launches += 1
        return cs

    def rope_store(self, qkv, num_heads, num_kv_heads, head_dim, positions, token_seq, inv_freq, style,
                   k_pages, v_pages, block_table, page_size, write_kv, q_out=None, cs_table=None):
        """Rotates q and k and stores k, v into the pages.  qkv [T, width] is rotated in place; qkv given
        as float32 partial sums [S, T, width] is summed, rotated, and q written to ``q_out`` [T, Hq*D].
        ``cs_table`` (from ``rope_table``) replaces the per-layer sine/cosine evaluation."""
        partial = qkv.dim() == 3
        T = qkv.shape[-2]
        stream = self._stream(qkv)
        vec_ok = head_dim % 4 == 0 and (inv_freq is None or (style == 0 and cs_table is not None)) and \
            (partial or (qkv.stride(0) % 4 == 0 and qkv.stride(1) == 1))
        if vec_ok:
            dst = q_out if partial else qkv
            self._check(self.lib.ttie_rope_store_vec(
                None if partial else _ptr(qkv), 0 if partial else qkv.stride(0), _ptr(qkv) if partial else None,
                qkv.shape[0] if partial else 0, qkv.stride(0) if partial else 0, T, num_heads, num_kv_heads, head_dim,
                _ptr(positions), _ptr(token_seq), None if inv_freq is None else _ptr(cs_table), _ptr(dst), dst.stride(0),
                _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1], page_size, k_pages.shape[0],
                1 if write_kv else 0, self._dt(dst), stream), "rope_store_vec")
        elif partial:
            self._check(self.lib.ttie_rope_store_partial(
                _ptr(qkv), qkv.shape[0], qkv.stride(0), T, num_heads, num_kv_heads, head_dim, _ptr(positions), _ptr(token_seq),
                _ptr(inv_freq), int(style), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], page_size, k_pages.shape[0], 1 if write_kv else 0, self._dt(q_out),
                stream), "rope_store_partial")
        else:
            self._check(self.lib.ttie_rope_store(_ptr(qkv), qkv.stride(0), T, num_heads, num_kv_heads, head_dim,
                                                 _ptr(positions), _ptr(token_seq), _ptr(inv_freq), int(style),
                                                 _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                                                 page_size, k_pages.shape[0], 1 if write_kv else 0, self._dt(qkv),
                                                 stream), "rope_store")
        self.launches += 1

    def attention_plan(self, dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size=None,
                       no_cluster_form=False):
        """Which attention kernel runs and how the key range is split: (kernel, num_splits,
        split_len).  bfloat16 with a head size that is a multiple of 16 up to 128, or 256, runs
        on tensor cores; everything else runs the general float32-arithmetic kernel.  The key
        range is split only when the query rows alone cannot fill the GPU.  Every layer of a step
        asks the same question, so the answers are kept.  ``no_cluster_form``: the thread-block-cluster decode form is left out
        of the choice (sigmoid weights, which every other kernel computes)."""
        key = (dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size, bool(no_cluster_form))
        plan = self._plans.get(key)
        if plan is None:
            if len(self._plans) >= 4096:
                self._plans.clear()
            plan = self._plans[key] = self._attention_plan(*key)
        return plan

    def _attention_plan(self, dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size, no_cluster_form=False):
        G = num_heads // num_kv_heads
        rows = max_q_len * G
        if (dtype == torch.bfloat16 and page_size is not None and head_dim > 128
                and self.lib.ttie_attn_tc_supported(head_dim, page_size)):
            return self._tc_wide_plan(num_seqs, num_kv_heads, rows, max_kv_len, max_q_len)
        if (dtype == torch.bfloat16 and page_size is not None and rows >= self.attn_tc_min_rows
                and self.lib.ttie_attn_tc_supported(head_dim, page_size)):
            # prompt portions: the tcgen05 kernel with two query tiles per CTA, uncut, where its CTAs fill half of the GPU
            # or more.  Below that the choice is between that kernel and the one-tile kernel (twice the CTAs), each with the
            # key range uncut or cut, by a cost model fitted to measurements (32 heads of 128; 1 to 8 portions of 128 to
            # 2,048 tokens behind 2,048 to 32,768 keys): waves of one CTA per SM at 3.5 us and 12 ns (one tile) or 17 ns (two)
            # per key, 2 us for the launch, and for cut ranges 3 us and the partial results' way through memory at 4 TB/s.
            # (512 tokens alone: one tile uncut, 14.3 against 18.4 us; the last 512 of 8,192: two tiles in two pieces, 83
            # against 103 one tile uncut and 134 two tiles uncut; the last 128 of 2,048: one tile in four pieces, 18.4
            # against 30.4 two tiles in two.)
            base = num_seqs * num_kv_heads * math.ceil(rows / 256)
            if base > self.num_sms // 2:
                return "tcpp", 1, 0
            return self._portion_pieces(num_seqs * num_kv_heads * rows, head_dim, max_kv_len,
                                        (("tc", num_seqs * num_kv_heads * math.ceil(rows / 128), 0.012), ("tcpp", base, 0.017)),
                                        max_kv_len >= 2 * max_q_len)
        if dtype == torch.bfloat16 and self.lib.ttie_attn_mma_supported(head_dim):
            # few rows per request: the tcgen05 kernel with the key range cut over CTAs where it applies (16 rows and more
            # per kv head, head size 64 or 128) - since it stages only the rows in use and sets itself up while its
            # predecessor finishes it is ahead of the decode form at every context (8 requests x 32 heads: 7.1 against
            # 10.7 us at 100 keys, 8.8 against 10.6 at 1,024, 9.6 against 10.7 at 2,048) -, else the decode form
            plan = self._tc_split_plan(num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size)
            if plan is not None:
                return plan
            plan = None if no_cluster_form else self._cluster_plan(num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len)
            if plan is not None:
                return plan
            kernel, tile_rows, unit, min_len = "mma", self.lib.ttie_attn_mma_tile_rows(max_q_len, num_heads, num_kv_heads), 64, 128
        else:
            kernel, tile_rows, unit, min_len = "simt", 32, 32, 32      # (one 32-key tile per CTA where the GPU has room: 10.6 us
                                                                      # against 21 for 200 keys in two pieces of 128)
        base = num_seqs * num_kv_heads * math.ceil(rows / tile_rows)
        if kernel == "mma" and rows <= 64:      # (one row tile per request and kv head: decoded tokens and the like)
            return self._mma_split_plan(base, head_dim, max_q_len, num_heads, num_kv_heads, max_kv_len)
        if base >= self.num_sms or max_kv_len <= min_len:
            return kernel, 1, 0
        # as many splits as fit one wave of resident CTAs, none shorter than min_len keys
        want = max(1, min(self.attn_target_ctas // base, math.ceil(max_kv_len / min_len)))
        split_len = math.ceil(math.ceil(max_kv_len / want) / unit) * unit
        num_splits = math.ceil(max_kv_len / split_len)
        return (kernel, num_splits, split_len) if num_splits > 1 else (kernel, 1, 0)

    def _portion_pieces(self, all_rows, head_dim, max_kv_len, kernels, may_cut):
        """The cheapest of ``kernels`` (name, CTAs per piece, us per key) and cuts of the key range for prompt portions whose
        CTAs fill less than half of the GPU: one wave of CTAs at 3.5 us + the keys of a piece, 2 us for the launch, and for
        a cut range 3 us and the partial results' way through memory at 4 TB/s.  A cut range stays within one wave; a
        portion that is most of its own context (``may_cut`` false) is not cut: behind the diagonal a piece has no work."""
        best, best_cost = (kernels[0][0], 1, 0), None
        for kernel, tiles, per_key in kernels:
            for want in range(1, (min(16, math.ceil(max_kv_len / 128)) if may_cut else 1) + 1):
                split_len = math.ceil(math.ceil(max_kv_len / want) / 128) * 128
                n = math.ceil(max_kv_len / split_len)
                if n != want or (n > 1 and tiles * n > self.num_sms):
                    continue                                         # (a cut range in several waves lost wherever it was measured)
                cost = math.ceil(tiles / self.num_sms) * (3.5 + min(split_len, max_kv_len) * per_key) + 2.0
                if n > 1:
                    cost += 3.0 + all_rows * (n * (4 * head_dim + 8) + 2 * head_dim) / 4e6
                if best_cost is None or cost < best_cost - 1e-9:
                    best, best_cost = ((kernel, n, split_len) if n > 1 else (kernel, 1, 0)), cost
        return best

    def _mma_split_plan(self, base, head_dim, max_q_len, num_heads, num_kv_heads, max_kv_len):
        """Pieces of the key range for the mma.sync tile loop, by a cost model fitted to measurements (head size 128,
        16-row tiles, 8 to 200 requests on 2 and 8 kv heads, 300 to 8,192 keys).  An SM holds a handful of the kernel's
        CTAs (5 at head size 128) and all of them together stream at a fixed rate, so the CTAs run in waves of
        ``resident``: a wave costs about 4.3 us and 74 ns per key of its pieces (58 ns when the wave fills less than a
        third of the GPU: a CTA alone on its SM runs faster), and 769 CTAs take as long as 1,480.  From three waves on the
        waves blur and the cost is proportional to the CTAs.  Merging costs 2 us.  Against picking the pieces by a fixed
        target of CTAs this is 16 % faster on average over those measurements and up to 70 % (24 requests x 8 kv heads at
        300 keys: 12.5 us in 3 pieces against 19.7 uncut; at 2,048 keys 54.6 against 71.4)."""
        key = (head_dim, max_q_len * (num_heads // num_kv_heads) <= 16, max_q_len * (num_heads // num_kv_heads) <= 32)
        per_sm = self._mma_per_sm.get(key)
        if per_sm is None:
            per_sm = self._mma_per_sm[key] = max(1, self.lib.ttie_attn_mma_ctas_per_sm(head_dim, max_q_len, num_heads, num_kv_heads))
        resident = per_sm * self.num_sms
        full_key = 0.0743 * (head_dim + 8) / 136

        def per_key(fill):
            return full_key * (0.78 + max(0.0, min(fill, 0.86) - 0.3) * 0.4)

        best, best_cost = ("mma", 1, 0), None
        shortest = 64 if max_q_len * (num_heads // num_kv_heads) <= 16 else 128      # (32 rows, 16 requests at 2,048 keys: 10.9 us in pieces of 128, 13.6 of 64)
        for want in range(1, min(128, math.ceil(max_kv_len / shortest)) + 1):
            split_len = math.ceil(math.ceil(max_kv_len / want) / 64) * 64
            n = math.ceil(max_kv_len / split_len)
            if n != want:
                continue
            ctas, keys = base * n, min(split_len, max_kv_len)
            if ctas >= 3 * resident:
                cost = ctas / resident * (4.3 + keys * full_key)
            else:
                whole, rest = divmod(ctas, resident)
                cost = whole * (4.3 + keys * full_key) + ((4.3 + keys * per_key(rest / resident)) if rest else 0.0)
            cost += 2.0 if n > 1 else 0.0
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = (("mma", n, split_len) if n > 1 else ("mma", 1, 0)), cost
        return best

    def _tc_wide_plan(self, num_seqs, num_kv_heads, rows, max_kv_len, max_q_len):
        """Head size 256: every step takes the prompt-portion tcgen05 kernel with one 128-row tile per CTA.  Steps of few
        rows (decoded tokens) have their key range cut by the cost model of the one-tile decode kernel, at 20 ns per key
        (8 heads on one kv head, 2 requests at 1,024 keys: 9.3 us in 8 pieces of 128 against 11.5 in 4; 96 requests at
        8,192 keys: 132 us in 3 pieces against 153 uncut).  Portions whose row tiles fill less than half of the GPU are cut
        by the portions' cost model at 21 ns per key (512 tokens behind 2,048 keys: 25.5 us in 4 pieces against 33.0 in 2)."""
        base = num_seqs * num_kv_heads * math.ceil(rows / 128)
        if rows <= 128:
            return self._one_per_sm_pieces("tcpp", base, max_kv_len, 0.020, waves_min_keys=640)
        if base > self.num_sms // 2:
            return "tcpp", 1, 0
        return self._portion_pieces(num_seqs * num_kv_heads * rows, 256, max_kv_len, (("tcpp", base, 0.021),),
                                    max_kv_len >= 2 * max_q_len)

    def _tc_split_plan(self, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size):
        """The tcgen05 kernel for steps with few query rows per request: the key range of every request is cut into
        pieces, one CTA each (the kernel takes a whole SM), and the merge kernel adds the pieces.  None where the head
        or page size is not the kernel's, the rows exceed one 128-row tile, or there are so few rows per kv head and so
        many requests that the mma.sync kernel's 16-row tiles waste less."""
        rows = max_q_len * (num_heads // num_kv_heads)
        base = num_seqs * num_kv_heads
        if (page_size is None or rows > 128 or head_dim > 128
                or not self.lib.ttie_attn_tc_supported(head_dim, page_size)):
            return None
        # 16 rows or fewer fill an eighth of the kernel's row tile: it still wins while the GPU is far from full (2 requests
        # x 8 kv heads at 300 keys: 8.0 us against 10.0 for the decode form), the tile loop's 16-row CTAs win beyond (32
        # requests x 2 kv heads at 2,048 keys: 19.6 us against 22.9)
        if rows <= 16 and (base > 32 or base * max_kv_len > (32768 if rows == 16 else 16384)):
            return None
        if rows < 32 and base > self.num_sms:
            return None              # (40 heads on 2 kv heads, 96 requests at 2,048 keys: 72.7 us uncut against 56.8 for the tile loop)
        if base > self.num_sms and max_kv_len < 1024:
            return None              # more requests than SMs with short contexts: the tile loop is ahead (measured at 512 keys)
        # The number of pieces by a cost model fitted to measurements (32 heads of 128 and 71 heads of 64 on one kv head, 2
        # to 200 requests, 300 to 8,192 keys).  CTAs run in waves of one per SM; a wave costs about 3.5 us to set up and
        # finish and 12.5 ns per key (more with more than 64 query rows); the launch costs 2 us, merging the pieces 2
        # (5.5 with more than 32 pieces, which the general merge kernel adds up).  So few requests get pieces down to 128
        # keys (2 requests at 1,024 keys: 7.7 us in 8 pieces against 8.9 in 4), and where the requests alone leave the
        # last wave half empty the key range is cut although every SM has a CTA already (96 requests at 8,192 keys: 81 us
        # in 3 pieces against 99 uncut; 200 requests: 165 in 2 against 194) - but into pieces of 1,280 keys at least:
        # shorter ones in several waves lose (200 requests at 1,024 keys: 43.6 us in 2 pieces against 34.8 uncut).
        return self._one_per_sm_pieces("tc", base, max_kv_len, 0.0125 * (1.15 if rows > 64 else 1.0))

    def _one_per_sm_pieces(self, kernel, base, max_kv_len, per_key, waves_min_keys=1280):
        """The cheapest cut of ``max_kv_len`` keys into pieces of a multiple of 128 keys for a kernel that runs one CTA per
        SM, ``base`` CTAs per piece: waves of ``num_sms`` CTAs at 3.5 us + ``per_key`` us per key of a piece, 2 us for the
        launch, 2 for merging (5.5 with more than 32 pieces); pieces that run in several waves hold ``waves_min_keys`` or more."""
        best, best_cost = (kernel, 1, 0), None
        for want in range(1, min(256, math.ceil(max_kv_len / 128)) + 1):
            split_len = math.ceil(math.ceil(max_kv_len / want) / 128) * 128
            n = math.ceil(max_kv_len / split_len)
            if n != want or (n > 1 and base * n > self.num_sms and split_len < waves_min_keys):
                continue                                             # (the same cut as a smaller count; short pieces in several waves)
            cost = (math.ceil(base * n / self.num_sms) * (3.5 + min(split_len, max_kv_len) * per_key) + 2.0
                    + (0.0 if n == 1 else 2.0 if n <= 32 else 5.5))
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = ((kernel, n, split_len) if n > 1 else (kernel, 1, 0)), cost
        return best

    def _clusters_active(self, head_dim, max_q_len, num_heads, num_kv_heads, groups, size):
        key = (head_dim, max_q_len * (num_heads // num_kv_heads) <= 16, groups, size)
        if key not in self._cluster_max:
            self._cluster_max[key] = self.lib.ttie_attn_cluster_active(head_dim, max_q_len, num_heads, num_kv_heads, groups, size)
        return self._cluster_max[key]

    def _cluster_plan(self, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len):
        """The decode form ("mma_c4" / "mma_c2": one thread-block cluster per request and kv head, 4 or 2 key
        groups per CTA) for steps whose requests bring few query rows: (kernel, cluster size, keys per CTA),
        or None where the tile loop serves better (many rows; a long context with too few requests to
        fill the GPU with clusters)."""
        rows = max_q_len * (num_heads // num_kv_heads)
        if rows > self.attn_cluster_max_rows:
            return None
        tile_rows = self.lib.ttie_attn_cluster_tile_rows(max_q_len, num_heads, num_kv_heads)
        base = num_seqs * num_kv_heads * math.ceil(rows / tile_rows)
        groups = 4 if max_kv_len > 128 else 2
        want = max(1, min(self.attn_cluster_max_size, (self.num_sms + base // 2) // base, math.ceil(max_kv_len / (64 * groups))))
        C = 1 << (want.bit_length() - 1)                       # a power of two
        while C > 1 and self._clusters_active(head_dim, max_q_len, num_heads, num_kv_heads, groups, C) < base:
            C //= 2                                            # all clusters of the step have to run at once
        if self._clusters_active(head_dim, max_q_len, num_heads, num_kv_heads, groups, C) < 1:
            return None
        split_len = math.ceil(math.ceil(max_kv_len / C) / 64) * 64
        # measured: the form pays while a warp walks few tiles; beyond that the tile loop with more, smaller CTAs
        # and a merge kernel is as fast or faster
        if split_len > self.attn_cluster_tiles_per_warp * 64 * groups:
            return None
        return f"mma_c{groups}", C, split_len

    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, k_pages, v_pages, block_table, page_size,
                        query_start_loc, seq_lens, num_seqs, max_q_len, max_kv_len, scale, window, out,
                        plan=None, softcap=0.0, chunk=0, weights="softmax", head_bias=None):
        """Causal attention of the step's query rows over the paged keys and values.  ``window`` > 0: a row at position p
        sees keys p - window + 1 .. p.  ``chunk`` > 0 (instead of a window): a row at position p sees the keys of its own
        chunk of ``chunk`` positions up to p, chunks counted from position 0 of the sequence.  ``softcap`` > 0: a score s
        (scale applied) becomes softcap * tanh(s / softcap) before mask and softmax.  ``weights`` "sigmoid": a visible key
        weighs sigmoid(score + head_bias[head]) (``head_bias`` float32 [num_heads] or None) and nothing is normalised over the
        keys; every kernel but the thread-block-cluster decode form computes them."""
        if weights not in ("softmax", "sigmoid"):
            raise KernelError(f"paged_attention: unknown kind of weights {weights!r}")
        sig = weights == "sigmoid"
        if chunk and window:
            raise KernelError("paged_attention: a window and a chunk size exclude each other")
        T = qkv.shape[0]
        if max_kv_len > block_table.shape[1] * page_size:
            raise KernelError(f"paged_attention: a block table of {block_table.shape[1]} pages of {page_size} keys cannot cover {max_kv_len} keys")
        kernel, num_splits, split_len = plan if plan is not None else self.attention_plan(
            qkv.dtype, num_seqs, num_heads, num_kv_heads, head_dim, max_q_len, max_kv_len, page_size, sig)
        if sig and kernel not in ("mma", "simt", "tc", "tcpp"):
            raise KernelError(f"paged_attention: sigmoid weights have no {kernel!r} kernel")
        if kernel in ("tc", "tcpp"):
            scratch = None
            if num_splits > 1:
                scratch = torch.empty((T * num_heads * num_splits * (head_dim + 2),), dtype=torch.float32, device=qkv.device)
            self._check(self.lib.ttie_paged_attention_tc_weights(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(block_table),
                block_table.shape[1], page_size, _ptr(query_start_loc), _ptr(seq_lens), _ptr(out), T, num_seqs, num_heads,
                num_kv_heads, head_dim, max_q_len, float(scale), float(softcap or 0.0), int(window), int(chunk), num_splits, split_len, _ptr(scratch),
                1 if kernel == "tcpp" else 0, 1 if sig else 0, _ptr(head_bias), self._stream(qkv)), "paged_attention_tc")
            self.launches += 2 if num_splits > 1 else 1
            return
        form = {"mma": 0, "mma_c2": 2, "mma_c4": 4}.get(kernel)
        scratch = None
        if num_splits > 1 and not form:
            scratch = torch.empty((T * num_heads * num_splits * (head_dim + 2),), dtype=torch.float32, device=qkv.device)
        if form is not None:
            self._check(self.lib.ttie_paged_attention_mma_weights(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                page_size, _ptr(query_start_loc), _ptr(seq_lens), _ptr(out), T, num_seqs, num_heads, num_kv_heads,
                head_dim, max_q_len, float(scale), float(softcap or 0.0), int(window), int(chunk), num_splits, split_len, _ptr(scratch),
                form, 1 if sig else 0, _ptr(head_bias), self._stream(qkv)), "paged_attention_mma")
            self.launches += 2 if (num_splits > 1 and not form) else 1
            return
        else:
            self._check(self.lib.ttie_paged_attention_weights(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                page_size, _ptr(query_start_loc), _ptr(seq_lens), _ptr(out), T, num_seqs, num_heads, num_kv_heads,
                head_dim, max_q_len, float(scale), float(softcap or 0.0), int(window), int(chunk), num_splits, split_len, _ptr(scratch),
                self._dt(qkv), 1 if sig else 0, _ptr(head_bias), self._stream(qkv)), "paged_attention")
        self.launches += 2 if num_splits > 1 else 1

    # ---- post-norm layers
    def scale_add_layernorm(self, resid, delta, alpha, weight, bias, eps, out=None, rows=None, num_rows=None, write_resid=True,
                            add_normed=False):
        """resid <- LayerNorm(alpha * resid + delta) * weight + bias over the 32-bit stream [R, d]; ``out`` (compute dtype, or
        None) receives a copy.  ``delta``: None, [R, d] or float32 partial sums [S, R, d].  With ``rows`` the rows are gathered
        into ``out`` [num_rows, d].  ``add_normed``: resid <- resid + LayerNorm(delta) * weight + bias instead (the norm sits on a
        sub-layer's output; ``alpha`` is not used)."""
        if add_normed and (delta is None or rows is not None):
            raise KernelError("scale_add_layernorm: add_normed needs a delta and takes no row list")
        d = resid.shape[1]
        R = resid.shape[0] if rows is None else int(num_rows)
        dp, pp, S, stride, ddt = None, None, 0, 0, 0
        if delta is not None:
            if delta.dim() == 3:
                pp, S, stride = delta.data_ptr(), delta.shape[0], delta.stride(0)
            else:
                dp, ddt = delta.data_ptr(), self._dt(delta)
        odt = self._dt(out) if out is not None else (0 if weight.dtype == torch.float32 and (delta is None or delta.dtype == torch.float32) else 1)
        self._check(self.lib.ttie_scale_add_layernorm(_ptr(resid), dp, ddt, pp, S, stride, _ptr(rows), _ptr(weight), _ptr(bias),
                                                      self._dt(weight), _ptr(out), odt, R, d, float(alpha), float(eps),
                                                      1 if (write_resid and rows is None) else 0, 1 if add_normed else 0,
                                                      self._stream(resid)),
                    "scale_add_layernorm")
        self.launches += 1

    def cast_rows(self, x32, dtype):
        """A copy of a float32 tensor in ``dtype``."""
        out = torch.empty(x32.shape, dtype=dtype, device=x32.device)
        self._check(self.lib.ttie_cast_rows(_ptr(x32), _ptr(out), x32.numel(), _DT[dtype], self._stream(x32)), "cast_rows")
        self.launches += 1
        return out

    # ---- latent attention
    def latent_store(self, proj, col0, rank, rot, norm_weight, eps, cs_table, positions, token_seq, pages, block_table, page_size):
        """Normalises (RMS, weight) the ``rank`` latent columns of ``proj`` from ``col0``, rotates the ``rot`` columns after
        them by the tokens' positions and stores the row into ``pages`` [pages, 1, page, width]."""
        T = proj.shape[0]
        self._check(self.lib.ttie_latent_store(_ptr(proj), proj.stride(0), int(col0), T, int(rank), int(rot), pages.shape[-1],
                                               _ptr(norm_weight), self._dt(norm_weight), float(eps), _ptr(cs_table), _ptr(positions),
                                               _ptr(token_seq), _ptr(pages), _ptr(block_table), block_table.shape[1], int(page_size),
                                               pages.shape[0], self._dt(proj), self._stream(proj)), "latent_store")
        self.launches += 1

    def latent_query(self, q, folded, num_heads, dim, rank, rot, width, cs_table):
        """[T, H, width] rows [folded query | rotated query part | zeros] from q [T, H * (dim + rot)] (a view with a row
        stride) and folded [H, T, rank]."""
        T = q.shape[0]
        out = torch.empty((T, num_heads * width), dtype=q.dtype, device=q.device)
        self._check(self.lib.ttie_latent_query(_ptr(q), q.stride(0), _ptr(folded), T, num_heads, dim, rank, rot, width, _ptr(cs_table),
                                               _ptr(out), self._dt(q), self._stream(q)), "latent_query")
        self.launches += 1
        return out

    def gate_heads(self, v, gate, num_heads, vdim, per_value=False):
        """out[t, h, :] = v[h, t, :] * sigmoid(gate[t, h]); v [H, T, vdim], gate a view [T, H] with a row stride.
        ``per_value``: gate is [T, H * vdim], one number per value."""
        T = gate.shape[0]
        out = torch.empty((T, num_heads * vdim), dtype=v.dtype, device=v.device)
        self._check(self.lib.ttie_gate_heads(_ptr(v), _ptr(gate), gate.stride(0), 1 if per_value else 0, T, num_heads, vdim, _ptr(out),
                                             self._dt(v), self._stream(v)), "gate_heads")
        self.launches += 1
        return out

    def rmsnorm_cols(self, proj, col0, width, weight, eps):
        """out[t] = proj[t, col0 : col0 + width] / sqrt(mean(.^2) + eps) * weight, [T, width] in proj's dtype (32-bit inside)."""
        T = proj.shape[0]
        out = torch.empty((T, width), dtype=proj.dtype, device=proj.device)
        self._check(self.lib.ttie_rmsnorm_cols(_ptr(proj), proj.stride(0), int(col0), T, int(width), _ptr(weight), self._dt(weight),
                                               float(eps), _ptr(out), self._dt(proj), self._stream(proj)), "rmsnorm_cols")
        self.launches += 1
        return out

    # ---- a causal convolution over time on the rows of the 32-bit residual stream
    def stream_conv(self, resid, conv_w, taps, tail, token_seq, query_start_loc, slot_ids, dtype, update_tail=False):
        """h[t] = sum_k conv_w[k] * x_(t - taps + 1 + k) per channel over the stream rows ``resid`` float32 [T, d]; ``conv_w``
        float32 tap-major [taps, d]; rows before the step come from ``tail`` float32 [slots + 1, taps - 1, d] (None with one
        tap).  Returns h [T, d] in ``dtype``.  ``conv_tail_update`` (given ``resid``) advances the state rows afterwards -
        or this call does, with ``update_tail``, which is only right for a step in which every request brings one token."""
        T, d = resid.shape
        out = torch.empty((T, d), dtype=dtype, device=resid.device)
        self._check(self.lib.ttie_stream_conv(_ptr(resid), T, d, int(taps), _ptr(conv_w), _ptr(tail), 0 if tail is None else tail.shape[0],
                                              _ptr(token_seq), _ptr(query_start_loc), _ptr(slot_ids), _ptr(out), _DT[dtype],
                                              1 if (update_tail and tail is not None) else 0, self._stream(resid)), "stream_conv")
        self.launches += 1
        return out

    def batched_linear(self, x, w, out_dtype=None):
        """y[b] = x[b] @ w[b].T for x [B, M, K] (any batch and row strides, unit inner stride) and w [B, N, K] contiguous
        -> [B, M, N] contiguous.  float32: this package's FFMA kernel; bfloat16: the library's batched product."""
        B, M, K = x.shape
        N = w.shape[1]
        if x.dtype == torch.float32:
            out = torch.empty((B, M, N), dtype=torch.float32, device=x.device)
            if x.stride(2) != 1 or w.stride(2) != 1:
                raise KernelError("batched_linear: inner strides must be 1")
            self._check(self.lib.ttie_gemm_f32_batched(_ptr(x), _ptr(w), _ptr(out), B, M, N, K, x.stride(1), w.stride(1), N,
                                                       x.stride(0), w.stride(0), M * N, self._stream(x)), "gemm_f32_batched")
            self.launches += 1
            return out
        if out_dtype is not None and out_dtype != x.dtype:
            return torch.bmm(x, w.transpose(1, 2), out_dtype=out_dtype)
        return torch.bmm(x, w.transpose(1, 2))

    # ---- recurrent block
    def causal_conv(self, xin, col0, width, taps, conv_w, conv_b, state, token_seq, query_start_loc, slot_ids, want_copy):
        """Per-channel causal convolution over the step's tokens (``conv_w`` tap-major [taps, width]); inputs before the
        step come from the state rows.
        Returns (u float32 [T, width], u in the compute dtype or None)."""
        T = xin.shape[0]
        u32 = torch.empty((T, width), dtype=torch.float32, device=xin.device)
        u_c = torch.empty((T, width), dtype=xin.dtype, device=xin.device) if want_copy else None
        self._check(self.lib.ttie_causal_conv(_ptr(xin), xin.stride(0), int(col0), T, width, taps, _ptr(conv_w), _ptr(conv_b),
                                              self._dt(conv_w), _ptr(state), state.shape[0], _ptr(token_seq), _ptr(query_start_loc),
                                              _ptr(slot_ids), _ptr(u32), _ptr(u_c), self._dt(xin), self._stream(xin)), "causal_conv")
        self.launches += 1
        return u32, u_c

    def rglru_scan(self, pre, gate_bias_r, gate_bias_i, lam, u32, xin, col_x, ypre, col_y, state, query_start_loc, slot_ids, num_seqs,
                   width, taps, block, decay_c, max_q_len, num_tokens):
        """The gated linear recurrence over the step's tokens from the state rows (advanced in place); returns S * gelu(y)
        in the compute dtype.  Portions longer than a chunk run the chunked form."""
        T = u32.shape[0]
        out = torch.empty((T, width), dtype=xin.dtype, device=xin.device)
        chunk = int(self.lib.ttie_rglru_chunk())
        ws = ab = None
        max_chunks = 0
        if max_q_len > 2 * chunk:
            max_chunks = num_tokens // chunk + num_seqs
            ws = torch.empty(2 * max_chunks + num_seqs, dtype=torch.int32, device=xin.device)
            ab = torch.empty((max_chunks, width, 3), dtype=torch.float32, device=xin.device)   # (prod a, input) per chunk, then the chunks' start states
        self._check(self.lib.ttie_rglru_scan(_ptr(pre), _ptr(gate_bias_r), _ptr(gate_bias_i), _ptr(lam), self._dt(lam), _ptr(u32),
                                             _ptr(xin), xin.stride(0), int(col_x), _ptr(ypre), ypre.stride(0), int(col_y),
                                             _ptr(state), state.shape[0], _ptr(query_start_loc), _ptr(slot_ids), num_seqs,
                                             _ptr(out), T, width, taps, block, float(decay_c), _ptr(ws), max_chunks, _ptr(ab),
                                             self._dt(xin), self._stream(xin)), "rglru_scan")
        self.launches += 4 if ws is not None else 1
        return out

    # ---- attention with a short convolution on its projections, partial rotation, another value size, gated heads
    def qkv_conv_rope_store(self, proj, num_heads, num_kv_heads, head_dim, v_dim, padded_dim, taps, conv_w, tail, positions, token_seq,
                            query_start_loc, slot_ids, cs_table, rot, style, k_pages, v_pages, block_table, page_size, write_kv,
                            norm_w=None, norm_eps=0.0, v_from_k=False, q_temp=None, row_inv=None):
        """From a step's projected rows ``proj`` [T, >= Hq*D + Hkv*D + Hkv*Dv] (columns [q | k | v]): the short causal
        convolution over time (``conv_w`` float32 tap-major [taps, channels]; ``tail`` float32 state rows
        [slots + 1, taps - 1, channels] with each request's last projected rows; ``taps`` 1 and ``conv_w`` None: none), the
        rotation of the first ``rot`` values of every q and k head (``style`` 0: pairs (2i, 2i+1), 1: pairs (i, i + rot/2);
        ``cs_table`` from ``rope_table``), and the store of k and v into the pages, rows padded with zeros to
        ``padded_dim``.  ``norm_w`` (float32 [2, head_dim]: the query heads' weights, then the key heads'): every q and k head
        is divided by its root mean square (``norm_eps`` inside the root) and multiplied by its weights, before the rotation.
        ``v_from_k``: ``proj`` has no v columns and a value head is its key head as it stands before norm and rotation.
        ``q_temp`` (coef, every): q at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).
        ``row_inv`` (float32 [T, 2] from ``proj_row_rms``): one norm over the whole q and one over the whole k projection
        instead of one per head; ``norm_w`` is then float32 [Hq*D + Hkv*D], a weight per channel.
        Returns q [T, Hq * padded_dim].  The state rows are advanced by ``conv_tail_update``."""
        T = proj.shape[0]
        q = torch.empty((T, num_heads * padded_dim), dtype=proj.dtype, device=proj.device)
        self._check(self.lib.ttie_qkv_conv_rope_store(
            _ptr(proj), proj.stride(0), T, num_heads, num_kv_heads, head_dim, v_dim, padded_dim, int(taps), _ptr(conv_w), _ptr(tail),
            0 if tail is None else tail.shape[0], _ptr(positions), _ptr(token_seq), _ptr(query_start_loc), _ptr(slot_ids),
            _ptr(cs_table), int(rot), int(style), _ptr(norm_w), float(norm_eps), _ptr(row_inv), 1 if v_from_k else 0,
            float(q_temp[0]) if q_temp else 0.0, int(q_temp[1]) if q_temp else 0,
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
            int(page_size), k_pages.shape[0], 1 if write_kv else 0, self._dt(proj), self._stream(proj)), "qkv_conv_rope_store")
        self.launches += 1
        return q

    def proj_row_rms(self, proj, nq, nk, eps):
        """float32 [T, 2]: 1 / sqrt(mean(x^2) + eps) over the first ``nq`` columns of every row of ``proj`` and over the next ``nk``."""
        T = proj.shape[0]
        inv = torch.empty((T, 2), dtype=torch.float32, device=proj.device)
        self._check(self.lib.ttie_proj_row_rms(_ptr(proj), proj.stride(0), T, int(nq), int(nk), float(eps), _ptr(inv), self._dt(proj),
                                               self._stream(proj)), "proj_row_rms")
        self.launches += 1
        return inv

    def conv_tail_update(self, proj, channels, taps, tail, query_start_loc, slot_ids, num_seqs):
        """Moves the last ``taps - 1`` projected rows of every request of the step into its state row (oldest first)."""
        if taps <= 1:
            return
        self._check(self.lib.ttie_conv_tail_update(_ptr(proj), proj.stride(0), int(channels), int(taps), _ptr(tail), tail.shape[0],
                                                   _ptr(query_start_loc), _ptr(slot_ids), int(num_seqs), self._dt(proj),
                                                   self._stream(proj)), "conv_tail_update")
        self.launches += 1

    def gate_head_rows(self, attn, gate, num_heads, v_dim, padded_dim, per_value=False):
        """out[t, h, :v_dim] = attn[t, h, :v_dim] * sigmoid(gate[t, h]); attn [T, H * padded_dim], gate a view [T, H] with a row
        stride, or None (then only the padding is dropped).  ``per_value``: gate is [T, H * v_dim], one number per value."""
        T = attn.shape[0]
        out = torch.empty((T, num_heads * v_dim), dtype=attn.dtype, device=attn.device)
        self._check(self.lib.ttie_gate_head_rows(_ptr(attn), _ptr(gate), 0 if gate is None else gate.stride(0), 1 if per_value else 0, T, num_heads, v_dim,
                                                 padded_dim, _ptr(out), self._dt(attn), self._stream(attn)), "gate_head_rows")
        self.launches += 1
        return out

    # ---- recurrent layers with a matrix state per head
    @staticmethod
    def matrix_state_pad(dim: int) -> int:
        """Key channels of a matrix-state row as the scan kernels lay it out: a power-of-two number of slices of 4 (heads of up
        to 128 key channels), 8 (up to 256) or 16 channels."""
        per_thread = 4 if dim <= 128 else 8 if dim <= 256 else 16
        slices = 1
        while slices * per_thread < dim:
            slices *= 2
        return slices * per_thread

    def token_shift_mix(self, x, mu, prev, token_seq, query_start_loc, slot_ids):
        """mixes[m, t] = x[t] + (x[t-1] - x[t]) * mu[m]; a request's first token of the step takes x[t-1] from its row of
        ``prev`` (float32 [slots + 1, d]).  x [T, d], mu float32 [M, d] -> [M, T, d]."""
        T, d = x.shape
        M = mu.shape[0]
        out = torch.empty((M, T, d), dtype=x.dtype, device=x.device)
        self._check(self.lib.ttie_token_shift_mix(_ptr(x), x.stride(0), T, d, M, _ptr(mu), _ptr(prev), prev.shape[0], _ptr(token_seq),
                                                  _ptr(query_start_loc), _ptr(slot_ids), _ptr(out), self._dt(x), self._stream(x)),
                    "token_shift_mix")
        self.launches += 1
        return out

    def wkv_decay(self, wlog, w0):
        """exp(-exp(wlog + w0)) in 32-bit: wlog float32 [T, H*dim] (a row stride allowed), w0 float32 [H*dim] -> [T, H*dim]."""
        T, HD = wlog.shape
        out = torch.empty((T, HD), dtype=torch.float32, device=wlog.device)
        self._check(self.lib.ttie_wkv_decay(_ptr(wlog), wlog.stride(0), _ptr(w0), _ptr(out), T, HD, self._stream(wlog)), "wkv_decay")
        self.launches += 1
        return out

    def wkv_scan(self, r, k, v, decay, u, state, x, prev, query_start_loc, slot_ids, num_seqs, num_heads, dim):
        """The time mix's recurrence over the step's tokens from the state rows ``state`` [slots + 1, H, dim, padded dim]
        (advanced in place): o_t = (S + diag(u) k v^T)^T r, then S <- diag(w) S + k v^T.  r, k, v [T, H*dim] views with one row
        stride; ``decay`` (w) float32 [T, H*dim] contiguous.  Also stores each request's last row of ``x`` into ``prev``.
        Returns o float32 [T, H*dim]."""
        T = r.shape[0]
        out = torch.empty((T, num_heads * dim), dtype=torch.float32, device=r.device)
        if not (r.stride(0) == k.stride(0) == v.stride(0)):
            raise KernelError("wkv_scan: r, k and v must share a row stride")
        self._check(self.lib.ttie_wkv_scan(_ptr(r), _ptr(k), _ptr(v), r.stride(0), _ptr(decay), _ptr(u),
                                           _ptr(state), state.shape[0], _ptr(x), x.stride(0), x.shape[1], _ptr(prev), prev.shape[0],
                                           _ptr(query_start_loc), _ptr(slot_ids), int(num_seqs), _ptr(out), num_heads, dim,
                                           self._dt(r), self._stream(r)), "wkv_scan")
        self.launches += 1
        return out

    def mlstm_gates(self, pre, m, n, query_start_loc, slot_ids, num_seqs, num_heads, cap):
        """Per token and head (state decay, input weight, exp(-running maximum)) from the gate pre-activations ``pre`` float32
        [T, 2H] (input gate's, then forget gate's), with log gates capped at ``cap``; the running maximum of every request
        moves in its row of ``m`` [slots + 1, H].  Also copies every request's normaliser state out of ``n``
        [slots + 1, H, padded dim] as it stands before the step.  Returns (float32 [T, H, 3], the copy [requests, H, padded dim])."""
        T = pre.shape[0]
        out = torch.empty((T, num_heads, 3), dtype=torch.float32, device=pre.device)
        snap = torch.empty((int(num_seqs), num_heads, n.shape[-1]), dtype=torch.float32, device=pre.device)
        self._check(self.lib.ttie_mlstm_gates(_ptr(pre), pre.stride(0), _ptr(m), m.shape[0], _ptr(query_start_loc), _ptr(slot_ids),
                                              int(num_seqs), _ptr(out), num_heads, float(cap), _ptr(n), _ptr(snap), n.shape[-1],
                                              self._stream(pre)), "mlstm_gates")
        self.launches += 1
        return out, snap

    def mlstm_scan(self, q, k, v, gates, S, n, n_before, query_start_loc, slot_ids, num_seqs, num_heads, dim, v_dim, q_scale):
        """The matrix memory's recurrence over the step's tokens from the state rows S [slots + 1, H, v_dim, padded dim] (advanced
        in place) and from ``n_before``, the copy of the normaliser state that ``mlstm_gates`` made (the new one is written
        into ``n`` [slots + 1, H, padded dim]).  q, k [T, H*dim], v [T, H*v_dim]: views with one row stride; ``gates`` from
        ``mlstm_gates``.  Returns o float32 [T, H*v_dim]."""
        T = q.shape[0]
        out = torch.empty((T, num_heads * v_dim), dtype=torch.float32, device=q.device)
        if not (q.stride(0) == k.stride(0) == v.stride(0)):
            raise KernelError("mlstm_scan: q, k and v must share a row stride")
        self._check(self.lib.ttie_mlstm_scan(_ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(gates), _ptr(S), _ptr(n), _ptr(n_before),
                                             S.shape[0], _ptr(query_start_loc), _ptr(slot_ids), int(num_seqs), _ptr(out), num_heads,
                                             dim, v_dim, float(q_scale), self._dt(q), self._stream(q)), "mlstm_scan")
        self.launches += 1
        return out

    def rotate_heads(self, src, heads, dim, cs_table, rot, style, scale_from=None, scale=1.0):
        """float32 [T, heads * dim]: the ``heads`` head rows of ``dim`` values at the start of every row of ``src`` (a view with a
        row stride), the first ``rot`` values of each rotated at the token's position (``cs_table`` from ``rope_table``;
        ``style`` 0: pairs (2i, 2i+1), 1: pairs (i, i + rot/2)), and the heads from ``scale_from`` on multiplied by ``scale``."""
        T = src.shape[0]
        out = torch.empty((T, heads * dim), dtype=torch.float32, device=src.device)
        self._check(self.lib.ttie_rotate_heads(_ptr(src), src.stride(0), T, int(heads), int(dim), int(rot), int(style), _ptr(cs_table),
                                               heads if scale_from is None else int(scale_from), float(scale), _ptr(out), self._dt(src),
                                               self._stream(src)), "rotate_heads")
        self.launches += 1
        return out

    def retention_scan(self, q, k, v, decay, S, query_start_loc, slot_ids, num_seqs, num_heads, dim, v_dim):
        """Retention's recurrence over the step's tokens from the state rows S [slots + 1, H, v_dim, padded dim] (advanced in
        place): S <- decay_h S + k v^T, o = S^T q.  q, k float32 [T, H*dim] views with one row stride; v [T, H*v_dim] in the
        compute dtype, a view with a row stride; ``decay`` float32 [H].  Returns o float32 [T, H*v_dim].

        A step that may hold a long prompt (the step's tokens less one for every other request: the host knows no more, and
        the number holds for a captured graph) is walked in ``parts`` (``retention_parts``) by two launches: the decay is a
        constant, so every part's own sum needs no other part and the parts' first states follow from those sums."""
        T = q.shape[0]
        out = torch.empty((T, num_heads * v_dim), dtype=torch.float32, device=q.device)
        if q.stride(0) != k.stride(0) or q.dtype != torch.float32 or k.dtype != torch.float32:
            raise KernelError("retention_scan: q and k must be float32 and share a row stride")
        parts = self.retention_parts(T, int(num_seqs), S[0].numel())
        scratch = torch.empty((int(num_seqs) * parts,) + tuple(S.shape[1:]), dtype=torch.float32, device=q.device) if parts > 1 else None
        self._check(self.lib.ttie_retention_scan(_ptr(q), _ptr(k), q.stride(0), _ptr(v), v.stride(0), _ptr(decay), _ptr(S), S.shape[0],
                                                 _ptr(query_start_loc), _ptr(slot_ids), int(num_seqs), _ptr(out), num_heads, dim, v_dim,
                                                 parts, _ptr(scratch), self._dt(v), self._stream(q)), "retention_scan")
        self.launches += 2 if parts > 1 else 1
        return out

    retention_part_tokens = 256             # a long prompt is walked in parts of about this many tokens,
    retention_max_parts = 16                # at most this many a request,
    retention_max_units = 64                # and requests x parts (state-sized scratch rows) at most this;
    retention_parts_state = 160 * 1024      # only where a request's state has at most this many elements

    def retention_parts(self, num_tokens: int, num_seqs: int, state_elems: int = 0) -> int:
        """Parts cost half as much work again (every part but the last is walked twice, once without read-out) and buy
        warps.  Measured on one 2,048-token prompt: a state of 8 heads x 128 x 128 takes 450 us in one piece (bound by the
        chain of tokens: twice the heads take the same time) and 320-350 us in 8 parts (bound by issued instructions: twice
        the heads take twice the time), so parts pay up to about 160 K state elements a request."""
        longest = num_tokens - (num_seqs - 1)                          # the most tokens one request of the step can bring
        if longest < 2 * self.retention_part_tokens or state_elems > self.retention_parts_state:
            return 1
        return max(1, min(self.retention_max_parts, longest // self.retention_part_tokens, self.retention_max_units // num_seqs))

    def head_norm_gate(self, o, gate, weight, num_heads, v_dim, eps, act):
        """out = o / rms(o over each head) * weight * act(gate); o float32 [T, H*v_dim], gate a view [T, H*v_dim] with a row
        stride, weight float32 [H*v_dim] or None (no weight); ``act``: "silu" or "sigmoid".  Returns the compute dtype of ``gate``."""
        T = o.shape[0]
        out = torch.empty((T, num_heads * v_dim), dtype=gate.dtype, device=o.device)
        self._check(self.lib.ttie_head_norm_gate(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), T, num_heads, v_dim, float(eps),
                                                 {"silu": 0, "sigmoid": 1}[act], _ptr(out), self._dt(gate), self._stream(o)),
                    "head_norm_gate")
        self.launches += 1
        return out

    # ---- elementwise functions between products
    _ACTIVATIONS = {"relu2": 0, "tanh": 1, "softcap": 2}

    def activation(self, x, kind, out_dtype=None, c=0.0, inplace=False):
        """f(x) elementwise in 32-bit: "relu2" (relu squared), "tanh", "softcap" (c * tanh(x / c)); x contiguous."""
        if not x.is_contiguous():
            raise KernelError("activation: the input must be contiguous")
        out = x if inplace else torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
        self._check(self.lib.ttie_activation(_ptr(x), _ptr(out), x.numel(), self._ACTIVATIONS[kind], float(c), self._dt(x),
                                             self._dt(out), self._stream(x)), "activation")
        self.launches += 1
        return out

    def linear_act(self, x, w, act):
        """act(x @ w.T) -> [M, N] in the compute dtype.  Where the weight-streaming product takes the step (few rows,
        bfloat16) the activation is its epilogue; else the product is followed by the activation kernel, in place."""
        if act == "relu2" and self._skinny_ok(x, w):
            M, K = x.shape
            N = w.shape[0]
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
            self._check(self.lib.ttie_skinny_gemm(_ptr(x), x.stride(0), _ptr(w), w.stride(0), None, _ptr(out), N, M, N, K,
                                                  math.ceil(K / 128) * 128, 4, 0, self._stream(x)), "skinny_gemm_relu2")
            self.launches += 1
            return out
        return self.activation(self.linear(x, w, None), act, inplace=True)

    # ---- gated linear units and routed experts
    def glu(self, gate_up, hidden, alpha=1.0, limit=0.0, shift=0.0):
        """g * sigmoid(alpha * g) * (u + shift) with optional clamps, gate_up = [g | u] per row -> [T, hidden]."""
        T = gate_up.shape[0]
        out = torch.empty((T, hidden), dtype=gate_up.dtype, device=gate_up.device)
        self._check(self.lib.ttie_glu(_ptr(gate_up), gate_up.stride(0), _ptr(out), T, hidden, float(alpha), float(limit or 0.0),
                                      float(shift), self._dt(gate_up), self._stream(gate_up)), "glu")
        self.launches += 1
        return out

    def moe_route(self, logits, groups, keep, group_top, top, scale, renorm=False, score="sigmoid", correction=None):
        """(expert ids int32 [T, top], weights float32 [T, top]) from float32 router logits [T, E] (rows may lie further apart
        than E).  ``score``: "sigmoid" per
        expert or "softmax" over all of them; ``correction`` float32 [E]: added to the scores for the choice only."""
        T, E = logits.shape
        idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
        wts = torch.empty((T, top), dtype=torch.float32, device=logits.device)
        self._check(self.lib.ttie_moe_route(_ptr(logits), logits.stride(0), T, E, groups, keep, group_top, top, float(scale), 1 if renorm else 0,
                                            {"sigmoid": 0, "softmax": 1}[score], _ptr(correction), _ptr(idx), _ptr(wts),
                                            self._stream(logits)), "moe_route")
        self.launches += 1
        return idx, wts

    def moe_plan(self, idx, num_experts, identity=0):
        """Sorts the (token, choice) pairs by expert on the device: a dict with ``pos_of_pair``, ``pair_of_pos``, ``offsets``,
        the row-tile table and its size bound.  The last ``identity`` of the ``num_experts`` own no matrices: their pairs are
        sorted behind the others and get no row tiles."""
        P = idx.numel()
        tile = int(self.lib.ttie_moe_tile_rows())
        max_tiles = P // tile + num_experts
        buf = torch.empty(2 * P + num_experts + 1 + 4 * max_tiles + 4, dtype=torch.int32, device=idx.device)
        plan = {"pos_of_pair": buf[:P], "pair_of_pos": buf[P:2 * P], "offsets": buf[2 * P:2 * P + num_experts + 1],
                "tiles": buf[2 * P + num_experts + 1:2 * P + num_experts + 1 + 4 * max_tiles], "meta": buf[-4:], "max_tiles": max_tiles,
                "pairs": P, "idx": idx, "real_experts": num_experts - int(identity)}
        self._check(self.lib.ttie_moe_plan(_ptr(idx), P, num_experts, num_experts - int(identity), max_tiles, _ptr(plan["offsets"]), _ptr(plan["pos_of_pair"]),
                                           _ptr(plan["pair_of_pos"]), _ptr(plan["tiles"]), _ptr(plan["meta"]), self._stream(idx)),
                    "moe_plan")
        self.launches += 1
        return plan

    grouped_few_rows = 64                   # (token, choice) pairs up to which the grouped product streams every tile's weights once

    def _library_grouped(self, x, w, plan, gather_div):
        """The library's grouped product (bfloat16, many rows): rows gathered into expert order, then one call whose group
        boundaries are read on the device.  None where it does not apply (sizes, or a build of the library without it)."""
        if self._grouped_mm is False or x.dtype != torch.bfloat16 or w.shape[1] % 8 or w.shape[2] % 8:
            return None
        if self._grouped_mm is None:
            self._grouped_mm = getattr(torch.nn.functional, "grouped_mm", None) or getattr(torch, "_grouped_mm", None) or False
            if self._grouped_mm is False:
                return None
        rows = x
        if gather_div:
            rows = torch.empty((plan["pairs"], x.shape[1]), dtype=x.dtype, device=x.device)
            self._check(self.lib.ttie_gather_rows(_ptr(x), x.stride(0), _ptr(plan["pair_of_pos"]), int(gather_div), plan["pairs"],
                                                  x.shape[1], _ptr(rows), self._dt(x), self._stream(x)), "gather_rows")
            self.launches += 1
        try:
            return self._grouped_mm(rows, w.transpose(1, 2), offs=plan["offsets"][1:w.shape[0] + 1])
        except (RuntimeError, TypeError, NotImplementedError):
            if torch.cuda.is_current_stream_capturing():
                raise
            self._grouped_mm = False                                    # this build has none for the device: the own kernel serves
            return None

    def linear_glu(self, x, w_gu, hidden, alpha=1.0, limit=0.0, shift=0.0):
        """The gated unit's activation of x @ [Wg; Wu].T -> [M, hidden].  With SwiGLU's constants this is ``linear_swiglu`` and
        its fused forms; with others, up to 8 rows run the weight-streaming product with the unit in its epilogue (where that
        form measured faster for the shape), more rows the product and the activation kernel."""
        if alpha == 1.0 and not limit and shift == 0.0:
            return self.linear_swiglu(x, w_gu, None, hidden)
        if x.dtype == torch.bfloat16 and self._skinny_ok(x, w_gu) and self._fused_few_rows_wins(x, w_gu, None, hidden):
            M, K = x.shape
            act = torch.empty((M, hidden), dtype=x.dtype, device=x.device)
            self._check(self.lib.ttie_skinny_gemm_glu(_ptr(x), x.stride(0), _ptr(w_gu), w_gu.stride(0), _ptr(act), hidden, M, hidden, K,
                                                      float(alpha), float(limit or 0.0), float(shift), self._stream(x)), "skinny_gemm_glu")
            self.launches += 1
            return act
        return self.glu(self.linear(x, w_gu, None), hidden, alpha, limit, shift)

    def grouped_glu(self, x, w_gu, plan, gather_div, hidden, alpha=1.0, limit=0.0, shift=0.0):
        """The experts' gate/up products over rows sorted by expert, then the gated unit: [pairs, hidden].  Few rows: one
        kernel (the unit in the weight-streaming product's epilogue); many: the grouped product and the activation kernel."""
        few = plan["pairs"] <= self.grouped_few_rows
        E, N, K = w_gu.shape
        vn = 4 if x.dtype == torch.float32 else 8
        if few and K % vn == 0 and x.stride(0) % vn == 0:
            out = torch.empty((plan["pairs"], hidden), dtype=x.dtype, device=x.device)
            self._check(self.lib.ttie_grouped_gemm(_ptr(x), x.stride(0), _ptr(plan["pair_of_pos"]) if gather_div else None, int(gather_div),
                                                   _ptr(w_gu), w_gu.stride(0), w_gu.stride(1), _ptr(out), hidden, _ptr(plan["tiles"]),
                                                   _ptr(plan["meta"]), plan["max_tiles"], N, K, self._dt(x), self._dt(out), 1, int(hidden),
                                                   float(alpha), float(limit or 0.0), float(shift), self._stream(x)), "grouped_gemm (gated)")
            self.launches += 1
            return out
        return self.glu(self.grouped_linear(x, w_gu, plan, gather_div), hidden, alpha, limit, shift)

    _ROW_ACTS = {None: 0, "relu2": 1}

    def grouped_act(self, x, w_up, plan, gather_div, act, row_scale=None):
        """The experts' up products over rows sorted by expert, with an activation behind them: row ``pos`` is
        ``act(s * (x[pair_of_pos[pos] // gather_div] @ w_up[e].T))`` -> [pairs, F] in the compute dtype.  ``row_scale`` float32
        [T, top]: s is the pair's routing weight - the weight goes in AHEAD of the expert (it multiplies the expert's input; the
        product being linear, it is applied to the 32-bit sums) -, None: 1.  ``act``: "relu2" or None.  Few rows, or 32-bit: the
        activation is the product's epilogue; many rows in bfloat16: the library's grouped product, then one pass in place."""
        E, N, K = w_up.shape
        code = self._ROW_ACTS[act]
        few = plan["pairs"] <= self.grouped_few_rows
        scale_of = plan["pair_of_pos"] if row_scale is not None else None
        if not few and x.dtype == torch.bfloat16:
            out = self._library_grouped(x, w_up, plan, gather_div)
            if out is not None:
                if code or row_scale is not None:
                    self._check(self.lib.ttie_row_scale_act(_ptr(out), out.stride(0), plan["pairs"], N, code, _ptr(row_scale), _ptr(scale_of),
                                                            self._dt(out), self._stream(out)), "row_scale_act")
                    self.launches += 1
                return out
        out = torch.empty((plan["pairs"], N), dtype=x.dtype, device=x.device)
        self._check(self.lib.ttie_grouped_gemm_act(_ptr(x), x.stride(0), _ptr(plan["pair_of_pos"]) if gather_div else None, int(gather_div),
                                                   _ptr(w_up), w_up.stride(0), w_up.stride(1), _ptr(out), N, _ptr(plan["tiles"]),
                                                   _ptr(plan["meta"]), plan["max_tiles"], N, K, self._dt(x), self._dt(out), 1 if few else 0,
                                                   0, 1.0, 0.0, 0.0, code, _ptr(row_scale), _ptr(scale_of), self._stream(x)),
                    "grouped_gemm (activation)")
        self.launches += 1
        return out

    def grouped_linear(self, x, w, plan, gather_div=0, out_dtype=None):
        """Rows sorted by expert times their expert's matrix: w [E, N, K]; row ``pos`` of the result is
        x[pair_of_pos[pos] // gather_div] @ w[e].T (``gather_div`` 0: x[pos]).  Few rows: a kernel that streams each tile's
        weights once; many rows in bfloat16: the library's grouped product (its result is bfloat16 whatever ``out_dtype``
        asks: it has no wider output); else (float32) FFMA tiles."""
        E, N, K = w.shape
        few = plan["pairs"] <= self.grouped_few_rows
        if not few and x.dtype == torch.bfloat16:
            out = self._library_grouped(x, w, plan, gather_div)
            if out is not None:
                return out
        out = torch.empty((plan["pairs"], N), dtype=out_dtype or x.dtype, device=x.device)
        self._check(self.lib.ttie_grouped_gemm(_ptr(x), x.stride(0), _ptr(plan["pair_of_pos"]) if gather_div else None, int(gather_div),
                                               _ptr(w), w.stride(0), w.stride(1), _ptr(out), N, _ptr(plan["tiles"]), _ptr(plan["meta"]),
                                               plan["max_tiles"], N, K, self._dt(x), self._dt(out), 1 if few else 0, 0, 1.0, 0.0, 0.0,
                                               self._stream(x)), "grouped_gemm")
        self.launches += 1
        return out

    def moe_combine(self, y, plan, wts, shared, num_tokens, dim, x=None, shared_gate=None):
        """float32 [T, d]: the weighted sum of each token's expert rows (+ the shared expert's output).  ``x`` [T, d] (compute
        dtype): the tokens' own rows, which an identity expert returns (a plan made with ``identity`` > 0 needs them).
        ``wts`` None: the rows are added as they are (their weights went in ahead of the experts).  ``shared_gate``: float32
        logits, one per token (a view with a row stride), whose sigmoid scales the shared expert's row."""
        out = torch.empty((num_tokens, dim), dtype=torch.float32, device=y.device)
        top = plan["idx"].shape[1]
        sdt = self._dt(shared) if shared is not None else self._dt(x) if x is not None else self._dt(y)
        identity = plan["real_experts"] < plan["offsets"].numel() - 1
        if identity and x is None:
            raise KernelError("moe_combine: identity experts return the tokens' own rows, which were not given")
        if shared_gate is not None and (shared is None or shared_gate.dtype != torch.float32):
            raise KernelError("moe_combine: a gate on the shared expert needs that expert's rows and 32-bit logits")
        self._check(self.lib.ttie_moe_combine_gated(_ptr(y), self._dt(y), _ptr(plan["pos_of_pair"]), _ptr(wts), _ptr(shared), num_tokens, dim,
                                                    top, _ptr(out), sdt, _ptr(plan["idx"]) if identity else None, plan["real_experts"],
                                                    _ptr(x) if identity else None, x.stride(0) if identity else 0, _ptr(shared_gate),
                                                    0 if shared_gate is None else shared_gate.stride(0), self._stream(y)),
                    "moe_combine")
        self.launches += 1
        return out

    def sample(self, logits, slot_ids, state, out, probs_out=None, ctas_per_row=0):
        """``ctas_per_row``: 0 = chosen from the vocabulary's size; 1, 2, 4 or 8 CTAs (a cluster) share a row."""
        R, V = logits.shape
        self._check(self.lib.ttie_sample_tuned(_ptr(logits), R, V, _ptr(slot_ids), _ptr(state), _ptr(out), _ptr(probs_out),
                                               int(ctas_per_row), self._stream(logits)), "sample")
        self.launches += 1


_OPS = {}


def get_ops(device="cuda:0") -> CudaOps:
    """The kernel library for ``device``; raises if it cannot be had."""
    key = str(torch.device(device))
    if key not in _OPS:
        _OPS[key] = CudaOps(device)
    return _OPS[key]
