"""The kernel set of the engine: thin Python wrappers around the C launchers.

Each method allocates its output with torch, checks dtypes and shapes, and passes raw
pointers and the current CUDA stream to the library. There is no fallback: constructing
``CudaOps`` fails if the library cannot be built or loaded or no CUDA device is present.

Matrix products in bfloat16 go through ``torch.matmul`` (cuBLAS), as the reference uses its
library's matrix product (nn.Linear, src/mlx_one/models/language/lfm2/reference_math.py:33-34);
in float32 they go through this library's own FMA kernel, which never uses a
reduced-precision mode.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch

from ..parts.base import NormedInput
from .build import KernelBuildError, library_path

_F32, _BF16 = 0, 1
_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong


class KernelError(RuntimeError):
    """A kernel launcher refused its arguments or a kernel reported a fault."""


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


class CudaOps:
    name = "cuda"

    def __init__(self, device: torch.device | str = "cuda:0", verbose: bool = True) -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelBuildError("the engine needs a CUDA device (sm_100a); it has no CPU path")
        try:
            self.lib = ctypes.CDLL(str(library_path(verbose=verbose)))
        except OSError as exc:
            raise KernelBuildError(f"cannot load the CUDA extension: {exc}") from exc
        self.lib.mlxone_last_error.restype = ctypes.c_char_p
        if self.lib.mlxone_abi_version() != 1:
            raise KernelBuildError("the CUDA extension is of another version; rebuild it")
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0
        self.tensor_core_attention = True
        self.skinny_products = True
        # A norm applied inside the product that consumes it (the skinny product reads the 32-bit
        # rows, all warps sharing the sums of squares, the norm's weights staged before the wait
        # for the kernel before it): no norm kernel, but every block reads rows of twice the size.
        # Decode steps of the 1.2B shape at 4096 keys: batch 1 / 2 / 4 / 6 0.578 / 0.588 / 0.615 /
        # 0.644 ms against 0.597 / 0.610 / 0.642 / 0.660 ms with the norm kernel; batch 8 0.68
        # against 0.67 ms, batch 16 0.95 against 0.89 ms. So up to `fused_norm_max_rows` rows.
        self.fused_norms = True
        self.fused_norm_max_rows = 6
        self.tcgen05_min_rows = 128
        self.tcgen05_attention = True     # prefill attention with tcgen05 where it takes the geometry
        # ... and with the keys of its few items cut into parts when a launch has fewer items than SMs
        self.prefill_key_splits = True
        # decode attention: key splits merged by a thread-block cluster through distributed shared
        # memory instead of a scratch buffer and a merge kernel (one launch fewer a layer), for up
        # to `cluster_merge_max_splits` splits. Measured inside the decode step of the 1.2B shape at
        # 4096 keys (the kernel before attention is the qkv product, whose blocks still hold their
        # SMs' shared memory when the clusters are placed): clusters of 2 and 3 (batch 20 to 32)
        # 1.004 against 1.036 ms and 1.08 against 1.12 ms; clusters of 8 at batch 8 take either
        # 19.5 or 31 us a launch where nine splits and the merge kernel take 17.5 + 3 us
        # (0.686 against 0.667 ms a step); clusters of 4 at batch 12 (16 rows, four of them
        # fillers) 37 against 23.6 us a launch, at batch 16 29 against 30 us.
        self.cluster_merge = True
        self.cluster_merge_max_splits = 3
        # a step of single tokens: q/k norm, rotation and the page write inside the decode
        # attention kernel instead of a kernel of their own before it
        self.fused_decode_attention = True
        # a mixed step's leading single-token requests go to the decode attention kernel when
        # there are at least this many of them
        self.split_singles_from = 1
        self.tcgen05_always = False       # tests: take the tcgen05 kernel whenever it can run
        self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # tcgen05 products (TMA + tensor memory) for more rows than the skinny kernel takes
        self.tcgen05_products = bool(self.lib.mlxone_gemm_tcgen05_available())
        # 33 to 128 rows: a tcgen05 product with swapped operands (weights as the 128-row operand,
        # K split over a thread-block cluster). Off: at 64 rows only w2 is faster than the library's
        # product (12.0 us against 13.3 us; in_proj 10.7 us against 6.9 us, w13 + SwiGLU 21.7 us
        # against 17.3 us), because a block's start and epilogue (about 8 us) are not hidden
        self.swapped_products = False
        self._swapped_rows = self.lib.mlxone_gemm_tcgen05_swapped_max_rows()
        self._skinny_rows = self.lib.mlxone_gemm_skinny_max_rows()
        # The skinny kernel takes up to 32 rows, but beyond 8 (more than one group of eight
        # tokens per tensor-core instruction) the library's product is faster: a decode step at
        # batch 16 takes 0.91 ms against 1.07 ms, at batch 32 0.98 ms against 1.91 ms
        self.skinny_max_rows = 8
        # With an epilogue of its own (SwiGLU, the residual add, the conv update) it is the faster
        # one up to 16 rows: out_proj 4.3 us against 5.7 us, w2 10.5 us against 13.0 us, w13 with
        # its gate 14.6 us against 12.9 us plus a gate kernel
        self.skinny_fused_max_rows = 16
        self._sample_scratch: torch.Tensor | None = None
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()

    # ------------------------------------------------------------------ plumbing

    def _stream(self) -> int:
        """The current stream's handle (the capture stream while a graph is captured). torch's
        raw query costs a fraction of building a Stream object, which a step would pay a
        hundred times."""
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _call(self, name: str, *args: Any) -> None:
        code = getattr(self.lib, name)(*args, _c_void_p(self._stream()))
        if code != 0:
            raise KernelError(self.lib.mlxone_last_error().decode())
        self.launches += 1

    def _need(self, tensor: torch.Tensor, dtype: torch.dtype, what: str) -> None:
        if tensor.dtype != dtype or not tensor.is_contiguous() or tensor.device != self.device:
            raise KernelError(f"{what} must be a contiguous {dtype} tensor on {self.device}, got "
                              f"{tensor.dtype} {tuple(tensor.shape)} on {tensor.device}")

    def set_dependent_launches(self, enabled: bool) -> None:
        """Programmatic dependent launches on the decode path: a kernel may start, and fetch
        its weights, while the one before it finishes."""
        self.lib.mlxone_set_pdl(1 if enabled else 0)

    ERRORS = {1: "a token id outside the vocabulary",
              2: "a key written to a position that has no page",
              3: "a key read from a position that has no page",
              9: "a wait inside a tcgen05 kernel that gave up"}

    def describe_error(self, code: int) -> KernelError:
        return KernelError(f"a kernel reported {self.ERRORS.get(code, f'code {code}')}")

    def check_errors(self) -> None:
        """Reads the device error flag (synchronises) and raises if a kernel set it."""
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise self.describe_error(code)

    # ------------------------------------------------------------------ size checks

    def check_attention_sizes(self, heads: int, kv_heads: int, head_dim: int) -> None:
        if heads % kv_heads:
            raise KernelError(f"{heads} query heads cannot share {kv_heads} key heads")
        if not 2 <= head_dim <= 512:
            raise KernelError(f"head size {head_dim} is outside 2..512")

    # ------------------------------------------------------------------ ops

    def embedding(self, ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        self._need(ids, torch.int32, "token ids")
        out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=self.device)
        self._call("mlxone_embedding", _c_void_p(_ptr(ids)), _c_void_p(_ptr(table)),
                   _c_void_p(_ptr(out)), _c_int(ids.numel()), _c_int(table.shape[1]),
                   _c_int(table.shape[0]), _c_int(_dtype_code(table.dtype)),
                   _c_void_p(_ptr(self.error_flag)))
        return out

    def add_rmsnorm(self, residual, delta, weight, eps, dtype):
        self._need(residual, torch.float32, "residual")
        self._need(weight, torch.float32, "norm weight")
        if delta is not None:
            self._need(delta, dtype, "delta")
            if delta.shape != residual.shape:
                raise KernelError("delta and residual differ in shape")
        rows, hidden = residual.shape
        if weight.numel() != hidden:
            raise KernelError(f"norm weight has {weight.numel()} entries, rows have {hidden}")
        out = torch.empty((rows, hidden), dtype=dtype, device=self.device)
        self._call("mlxone_add_rmsnorm", _c_void_p(_ptr(residual)), _c_void_p(_ptr(delta)),
                   _c_void_p(_ptr(weight)), _c_void_p(_ptr(out)), _c_int(rows), _c_int(hidden),
                   _c_float(eps), _c_int(_dtype_code(dtype)))
        return out

    def gather_rows(self, residual, delta, rows):
        self._need(residual, torch.float32, "residual")
        self._need(rows, torch.int32, "rows")
        count, hidden = rows.numel(), residual.shape[1]
        picked = torch.empty((count, hidden), dtype=torch.float32, device=self.device)
        picked_delta = None
        code = _F32
        if delta is not None:
            picked_delta = torch.empty((count, hidden), dtype=delta.dtype, device=self.device)
            code = _dtype_code(delta.dtype)
        self._call("mlxone_gather_rows", _c_void_p(_ptr(residual)), _c_void_p(_ptr(delta)),
                   _c_void_p(_ptr(rows)), _c_void_p(_ptr(picked)), _c_void_p(_ptr(picked_delta)),
                   _c_int(count), _c_int(hidden), _c_int(residual.shape[0]), _c_int(code))
        return picked, picked_delta

    # epilogues of the skinny product
    _STORE, _SWIGLU, _ADD, _STORE_F32 = 0, 1, 2, 3

    def _skinny(self, a, w, fused=False) -> bool:
        """Whether a[M, K] @ w[N, K]^T goes to the weight-streaming kernel: bfloat16, few rows,
        16-byte aligned rows. Everything else goes to the library product. ``fused``: the
        product has an epilogue that the library's product would need another kernel for."""
        most = max(self.skinny_max_rows, self.skinny_fused_max_rows) if fused else self.skinny_max_rows
        return (self.skinny_products and a.dtype == torch.bfloat16
                and 0 < a.shape[0] <= min(self._skinny_rows, most)
                and a.shape[1] % 8 == 0
                and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def enable_tcgen05(self, enabled: bool = True) -> bool:
        """Routes bfloat16 products with more rows than the skinny kernel takes to the
        tcgen05 kernel (TMA loads, accumulator in tensor memory) instead of the library."""
        self.tcgen05_products = bool(enabled) and bool(self.lib.mlxone_gemm_tcgen05_available())
        if not self.tcgen05_products:
            self.swapped_products = False
        return self.tcgen05_products

    def _tcgen05(self, a, w, epilogue=0) -> bool:
        """Whether a[M, K] @ w[N, K]^T goes to the tcgen05 kernel. It needs 16-byte aligned
        rows and at least 128 rows (its tiles are 128 x 256 and each persistent block walks
        whole tiles), and it is chosen where it is faster than the library's product plus the
        kernel that the library's product then needs: with the fused SwiGLU epilogue, which
        saves a pass over the widest activation (2048 rows: 100 us against 153 us; 512 rows: 35
        against 41), when its tiles fill the SMs to 60 %. Plain products and products added into
        the residual stream go to the library, which is faster at every row count measured
        (2048 rows: in_proj 37.7 us against 45.3, qkv 20.7 against 30.8, out_proj 14.8 against
        24.8 with the residual epilogue, w2 47 against 62; 8192 rows: 142 / 73 / 49 / 181 us
        against 156 / 82 / 77 / 244); their result is added by the next norm kernel."""
        if not (self.tcgen05_products and a.dtype == torch.bfloat16
                and a.shape[0] >= self.tcgen05_min_rows
                and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1
                and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            return False
        if self.tcgen05_always:
            return True
        if epilogue != self._SWIGLU:
            return False
        tiles = -(-a.shape[0] // 128) * -(-(w.shape[0] // 2) // 128)
        evenness = tiles / (-(-tiles // self._sm_count) * self._sm_count)
        return evenness >= 0.6

    def _tcgen05_call(self, a, w, bias, out, ldo, epilogue) -> None:
        self._call("mlxone_gemm_tcgen05", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                   _c_void_p(_ptr(w)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(ldo),
                   _c_int(a.shape[0]), _c_int(w.shape[0]), _c_int(a.shape[1]), _c_int(epilogue),
                   _c_void_p(_ptr(self.error_flag)))

    def _swapped(self, a, w) -> bool:
        """Whether a[M, K] @ w[N, K]^T goes to the tcgen05 product with swapped operands: more
        rows than the skinny kernel takes, at most 128, 16-byte aligned rows."""
        return (self.swapped_products and a.dtype == torch.bfloat16
                and min(self._skinny_rows, self.skinny_max_rows) < a.shape[0] <= self._swapped_rows
                and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1
                and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def _swapped_call(self, a, w, bias, out, ldo, epilogue) -> None:
        self._call("mlxone_gemm_tcgen05_swapped", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                   _c_void_p(_ptr(w)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(ldo),
                   _c_int(a.shape[0]), _c_int(w.shape[0]), _c_int(a.shape[1]), _c_int(epilogue),
                   _c_void_p(_ptr(self.error_flag)))

    def _skinny_call(self, a, w, bias, out, ldo, epilogue) -> None:
        self._call("mlxone_gemm_skinny", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                   _c_void_p(_ptr(w)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(ldo),
                   _c_int(a.shape[0]), _c_int(w.shape[0]), _c_int(a.shape[1]), _c_int(epilogue))

    def _check_product(self, a, w) -> None:
        if a.dtype != w.dtype:
            raise KernelError(f"matrix product of {a.dtype} with {w.dtype}")
        if a.dim() != 2 or w.dim() != 2 or w.shape[1] != a.shape[1]:
            raise KernelError(f"matrix product of {tuple(a.shape)} with {tuple(w.shape)}^T")

    # ---- norms applied inside the product that consumes them

    def can_fuse_norm(self, residual, dtype) -> bool:
        """Whether RMSNorm(residual) can be applied by the skinny product while it loads its
        input (bfloat16, up to 16 rows, the rows fit into shared memory)."""
        return (self.fused_norms and self.skinny_products and dtype == torch.bfloat16
                and residual.shape[0] <= self.fused_norm_max_rows
                and residual.dtype == torch.float32 and residual.is_contiguous()
                and bool(self.lib.mlxone_gemm_skinny_norm_fits(residual.shape[0], residual.shape[1])))

    def _normed_call(self, a, w, bias, out, ldo, epilogue) -> None:
        self._need(w, torch.bfloat16, "w")
        if w.shape[1] != a.residual.shape[1]:
            raise KernelError(f"matrix product of {tuple(a.shape)} with {tuple(w.shape)}^T")
        self._call("mlxone_gemm_skinny_norm", _c_void_p(_ptr(a.residual)),
                   _c_int(a.residual.stride(0)), _c_void_p(_ptr(a.weight)), _c_float(a.eps),
                   _c_void_p(_ptr(w)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(ldo),
                   _c_int(a.shape[0]), _c_int(w.shape[0]), _c_int(a.shape[1]), _c_int(epilogue))

    def linear(self, a, w, bias=None, out_dtype=None):
        """a[M, K] @ w[N, K]^T (+ bias[N], float32). ``out_dtype``: a's dtype, or float32."""
        if isinstance(a, NormedInput):
            out_dtype = out_dtype or a.dtype
            out = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype, device=self.device)
            self._normed_call(a, w, bias, out, w.shape[0],
                              self._STORE_F32 if out_dtype == torch.float32 else self._STORE)
            return out
        self._check_product(a, w)
        out_dtype = out_dtype or a.dtype
        m, k = a.shape
        n = w.shape[0]
        if a.dtype == torch.float32:
            self._need(a, torch.float32, "a")
            self._need(w, torch.float32, "w")
            out = torch.empty((m, n), dtype=torch.float32, device=self.device)
            self._call("mlxone_gemm_f32", _c_void_p(_ptr(a)), _c_int(k), _c_void_p(_ptr(w)),
                       _c_int(k), _c_void_p(_ptr(bias)), _c_void_p(_ptr(out)), _c_int(n),
                       _c_int(m), _c_int(n), _c_int(k))
            return out
        if self._skinny(a, w):
            out = torch.empty((m, n), dtype=out_dtype, device=self.device)
            self._skinny_call(a, w, bias, out, n,
                              self._STORE_F32 if out_dtype == torch.float32 else self._STORE)
            return out
        if self._swapped(a, w):
            out = torch.empty((m, n), dtype=out_dtype, device=self.device)
            self._swapped_call(a, w, bias, out, n,
                               self._STORE_F32 if out_dtype == torch.float32 else self._STORE)
            return out
        if self._tcgen05(a, w, self._STORE):
            out = torch.empty((m, n), dtype=out_dtype, device=self.device)
            self._tcgen05_call(a, w, bias, out, n,
                               self._STORE_F32 if out_dtype == torch.float32 else self._STORE)
            return out
        if out_dtype == torch.float32:
            out = torch.mm(a, w.t(), out_dtype=torch.float32)
        else:
            out = torch.mm(a, w.t())
        if bias is not None:
            self._call("mlxone_add_bias", _c_void_p(_ptr(out)), _c_void_p(_ptr(bias)), _c_int(m),
                       _c_int(n), _c_int(_dtype_code(out.dtype)))
        return out

    def linear_swiglu(self, a, gate_up):
        """silu(a @ gate^T) * (a @ up^T) with gate_up = [gate rows; up rows]: one kernel for
        few rows, else a product followed by the gate kernel."""
        if isinstance(a, NormedInput):
            width = gate_up.shape[0] // 2
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._normed_call(a, gate_up, None, out, width, self._SWIGLU)
            return out
        self._check_product(a, gate_up)
        if self._skinny(a, gate_up, fused=True):
            width = gate_up.shape[0] // 2
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._skinny_call(a, gate_up, None, out, width, self._SWIGLU)
            return out
        if self._swapped(a, gate_up):
            width = gate_up.shape[0] // 2
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._swapped_call(a, gate_up, None, out, width, self._SWIGLU)
            return out
        if self._tcgen05(a, gate_up, self._SWIGLU):
            width = gate_up.shape[0] // 2
            out = torch.empty((a.shape[0], width), dtype=a.dtype, device=self.device)
            self._tcgen05_call(a, gate_up, None, out, width, self._SWIGLU)
            return out
        return self.swiglu(self.linear(a, gate_up))

    def linear_add(self, a, w, bias, residual):
        """Adds a @ w^T (+ bias) to the float32 ``residual``. Returns None if it was added in
        place (few rows: the product's epilogue does it), else the product, which the caller
        adds with the next norm."""
        self._check_product(a, w)
        if self._skinny(a, w, fused=True):
            self._need(residual, torch.float32, "residual")
            self._skinny_call(a, w, bias, residual, residual.shape[1], self._ADD)
            return None
        if self._swapped(a, w):
            self._need(residual, torch.float32, "residual")
            self._swapped_call(a, w, bias, residual, residual.shape[1], self._ADD)
            return None
        if self._tcgen05(a, w, self._ADD):
            self._need(residual, torch.float32, "residual")
            self._tcgen05_call(a, w, bias, residual, residual.shape[1], self._ADD)
            return None
        return self.linear(a, w, bias)

    def swiglu(self, gate_up):
        rows, twice = gate_up.shape
        out = torch.empty((rows, twice // 2), dtype=gate_up.dtype, device=self.device)
        self._call("mlxone_swiglu", _c_void_p(_ptr(gate_up)), _c_void_p(_ptr(out)), _c_int(rows),
                   _c_int(twice // 2), _c_int(_dtype_code(gate_up.dtype)))
        return out

    def short_conv(self, bcx, *, kernel, bias, taps, ctx, view, write):
        tokens, triple = bcx.shape
        hidden = triple // 3
        self._need(bcx, view.state.dtype, "bcx")
        self._need(kernel, torch.float32, "conv kernel")
        out = torch.empty((tokens, hidden), dtype=bcx.dtype, device=self.device)
        if ctx.max_portion == 1 and tokens == ctx.requests:
            # decode: output and state update in one kernel
            self._call("mlxone_short_conv_decode", _c_void_p(_ptr(bcx)), _c_void_p(_ptr(kernel)),
                       _c_void_p(_ptr(bias)), _c_void_p(_ptr(view.state)),
                       _c_void_p(_ptr(view.slots)), _c_void_p(_ptr(ctx.history)),
                       _c_void_p(_ptr(out)), _c_int(tokens), _c_int(hidden), _c_int(taps),
                       _c_int(1 if write else 0), _c_int(_dtype_code(bcx.dtype)))
            return out
        self._call("mlxone_short_conv", _c_void_p(_ptr(bcx)), _c_void_p(_ptr(kernel)),
                   _c_void_p(_ptr(bias)), _c_void_p(_ptr(view.state)), _c_void_p(_ptr(view.slots)),
                   _c_void_p(_ptr(ctx.token_request)), _c_void_p(_ptr(ctx.request_start)),
                   _c_void_p(_ptr(ctx.history)), _c_void_p(_ptr(out)), _c_int(tokens),
                   _c_int(ctx.requests), _c_int(hidden), _c_int(taps), _c_int(1 if write else 0),
                   _c_int(_dtype_code(bcx.dtype)))
        return out

    def linear_short_conv(self, a, w, w_bias, *, kernel, bias, taps, ctx, view, write):
        """short_conv(linear(a, w, w_bias)): for a decode step of few rows one kernel, the
        convolution's update being the product's epilogue; else the two operations."""
        fits = (ctx.max_portion == 1 and a.shape[0] == ctx.requests and taps <= 4
                and w.shape[0] % 3 == 0 and view.state.dtype == torch.bfloat16)
        if (isinstance(a, NormedInput) and fits and self.lib.mlxone_gemm_skinny_conv_norm_fits(
                _c_int(a.shape[0]), _c_int(a.shape[1]))):
            # the norm while the rows are loaded, the product, the convolution's update: one kernel
            self._need(w, torch.bfloat16, "w")
            self._need(kernel, torch.float32, "conv kernel")
            if w.shape[1] != a.residual.shape[1]:
                raise KernelError(f"matrix product of {tuple(a.shape)} with {tuple(w.shape)}^T")
            hidden = w.shape[0] // 3
            out = torch.empty((a.shape[0], hidden), dtype=a.dtype, device=self.device)
            self._call("mlxone_gemm_skinny_conv_norm", _c_void_p(_ptr(a.residual)),
                       _c_int(a.residual.stride(0)), _c_void_p(_ptr(a.weight)), _c_float(a.eps),
                       _c_void_p(_ptr(w)), _c_void_p(_ptr(w_bias)), _c_void_p(_ptr(out)),
                       _c_int(a.shape[0]), _c_int(hidden), _c_int(a.shape[1]),
                       _c_void_p(_ptr(kernel)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(view.state)),
                       _c_void_p(_ptr(view.slots)), _c_void_p(_ptr(ctx.history)), _c_int(taps),
                       _c_int(1 if write else 0))
            return out
        if not isinstance(a, NormedInput) and fits and self._skinny(a, w, fused=True):
            self._check_product(a, w)
            self._need(kernel, torch.float32, "conv kernel")
            hidden = w.shape[0] // 3
            out = torch.empty((a.shape[0], hidden), dtype=a.dtype, device=self.device)
            self._call("mlxone_gemm_skinny_conv", _c_void_p(_ptr(a)), _c_int(a.stride(0)),
                       _c_void_p(_ptr(w)), _c_void_p(_ptr(w_bias)), _c_void_p(_ptr(out)),
                       _c_int(a.shape[0]), _c_int(hidden), _c_int(a.shape[1]),
                       _c_void_p(_ptr(kernel)), _c_void_p(_ptr(bias)), _c_void_p(_ptr(view.state)),
                       _c_void_p(_ptr(view.slots)), _c_void_p(_ptr(ctx.history)), _c_int(taps),
                       _c_int(1 if write else 0))
            return out
        return self.short_conv(self.linear(a, w, w_bias), kernel=kernel, bias=bias, taps=taps,
                               ctx=ctx, view=view, write=write)

    def qk_norm_rope_store(self, qkv, *, heads, kv_heads, head_dim, q_weight, k_weight, eps,
                           rotary, ctx, view, write):
        tokens = qkv.shape[0]
        self._need(qkv, view.kv.dtype, "qkv")
        if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
            raise KernelError("qkv width does not match the head counts")
        inv_freq, rotary_dim = (None, 0) if rotary is None else rotary
        q = torch.empty((tokens, heads, head_dim), dtype=qkv.dtype, device=self.device)
        pages = view.kv.shape[1]
        self._call("mlxone_qk_prep", _c_void_p(_ptr(qkv)), _c_void_p(_ptr(q_weight)),
                   _c_void_p(_ptr(k_weight)), _c_float(0.0 if eps is None else eps),
                   _c_void_p(_ptr(inv_freq)), _c_int(rotary_dim), _c_void_p(_ptr(ctx.positions)),
                   _c_void_p(_ptr(ctx.token_request)), _c_void_p(_ptr(q)),
                   _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(view.block_table)),
                   _c_int(view.block_table.shape[1]), _c_int(view.page_size), _c_int(pages),
                   _c_int(tokens), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
                   _c_int(1 if write else 0), _c_int(_dtype_code(qkv.dtype)),
                   _c_void_p(_ptr(self.error_flag)))
        return q

    def qkv_attention(self, qkv, *, heads, kv_heads, head_dim, q_weight, k_weight, eps, rotary,
                      scale, window, ctx, view, write):
        """From the fused projection qkv [tokens, (heads + 2 kv_heads) * head_dim] to the mixed
        heads [tokens, heads * head_dim]: per-head norm of queries and keys, rotation, keys and
        values appended to the pages, attention. A step of single tokens in bfloat16 whose head
        size is a multiple of 32 and whose rotation covers the whole head (or is none) runs as
        one kernel; everything else as the preparation kernel followed by attention."""
        tokens = qkv.shape[0]
        inv_freq, rotary_dim = (None, 0) if rotary is None else rotary
        if (self.fused_decode_attention and qkv.dtype == torch.bfloat16
                and ctx.max_portion == 1 and tokens == ctx.requests
                and self.tensor_core_attention
                and self.lib.mlxone_attention_decode_fused_supports(_c_int(head_dim))
                and (inv_freq is None or rotary_dim == head_dim)
                and (q_weight is None) == (k_weight is None)):
            self._need(qkv, view.kv.dtype, "qkv")
            if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
                raise KernelError("qkv width does not match the head counts")
            out = torch.empty((tokens, heads * head_dim), dtype=qkv.dtype, device=self.device)
            width = view.block_table.shape[1]
            splits, partial = self._decode_plan(tokens, heads, kv_heads, head_dim, width, window,
                                                view)
            self._call("mlxone_attention_decode_fused", _c_void_p(_ptr(qkv)),
                       _c_void_p(_ptr(q_weight)), _c_void_p(_ptr(k_weight)),
                       _c_float(0.0 if eps is None else eps), _c_void_p(_ptr(inv_freq)),
                       _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(view.block_table)), _c_int(width),
                       _c_int(view.page_size), _c_int(view.kv.shape[1]),
                       _c_void_p(_ptr(ctx.positions)), _c_void_p(_ptr(out)),
                       _c_void_p(_ptr(partial)), _c_int(tokens), _c_int(heads), _c_int(kv_heads),
                       _c_int(head_dim), _c_int(splits), _c_float(scale), _c_int(window or 0),
                       _c_int(1 if write else 0), _c_void_p(_ptr(self.error_flag)))
            if partial is not None:
                self.launches += 1          # the merge kernel
            return out
        q = self.qk_norm_rope_store(qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                    q_weight=q_weight, k_weight=k_weight, eps=eps, rotary=rotary,
                                    ctx=ctx, view=view, write=write)
        return self.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                    scale=scale, window=window, ctx=ctx, view=view)

    def paged_attention(self, q, *, heads, kv_heads, head_dim, scale, window, ctx, view):
        """Attention of every token over its request's pages. bfloat16 with a head size that
        is a multiple of 16 up to 128 runs on tensor cores: the split-key decode kernel when
        every request brings one token, else the prefill kernel. Everything else (float32,
        other head sizes) runs the general kernel."""
        tokens = q.shape[0]
        out = torch.empty((tokens, heads * head_dim), dtype=q.dtype, device=self.device)
        width = view.block_table.shape[1]
        pages = view.kv.shape[1]
        code = _dtype_code(q.dtype)
        if self.tensor_core_attention and self.lib.mlxone_attention_mma_supports(head_dim, code):
            if ctx.max_portion == 1 and tokens == ctx.requests:
                self._decode_attention(q, out, ctx.requests, heads, kv_heads, head_dim, scale,
                                       window, ctx, view)
                return out
            # The decodes at the head of a mixed step go to the split-key kernel, which reads
            # each request's keys once for all its query heads; as one-token portions in the
            # prefill kernel they would each fill a tile of 64 or 128 query rows with one row.
            singles = min(getattr(ctx, "leading_single", 0), ctx.requests)
            if singles < self.split_singles_from:
                singles = 0
            if singles:
                self._decode_attention(q, out, singles, heads, kv_heads, head_dim, scale, window,
                                       ctx, view)
            # the other requests: the tables, starts and histories from request ``singles`` on
            # (token numbers in request_start stay those of the whole step)
            rest = ctx.requests - singles
            table = view.block_table[singles:]
            starts, history = ctx.request_start[singles:], ctx.history[singles:]
            if (self.tcgen05_attention and q.dtype == torch.bfloat16
                    and self.lib.mlxone_attention_tcgen05_supports(
                        _c_int(head_dim), _c_int(heads), _c_int(kv_heads), _c_int(view.page_size))):
                # few query tiles (a prompt's portion beside a step's decodes): their keys are
                # cut into parts that run side by side, and a merge follows
                bound = min(ctx.max_context, width * view.page_size)
                if window:
                    bound = min(bound, window + ctx.max_portion)
                splits = 1
                if self.prefill_key_splits:
                    splits = self.lib.mlxone_attention_tcgen05_splits(
                        _c_int(tokens - singles), _c_int(rest), _c_int(heads), _c_int(kv_heads),
                        _c_int(bound))
                partial = None
                if splits > 1:
                    partial = torch.empty(tokens * heads * splits * (head_dim + 2),
                                          dtype=torch.float32, device=self.device)
                self._call("mlxone_attention_prefill_tcgen05", _c_void_p(_ptr(q)),
                           _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(table)),
                           _c_int(width), _c_int(view.page_size), _c_int(pages),
                           _c_void_p(_ptr(starts)), _c_void_p(_ptr(history)),
                           _c_void_p(_ptr(out)), _c_int(tokens), _c_int(rest),
                           _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_float(scale),
                           _c_int(window or 0), _c_int(splits), _c_void_p(_ptr(partial)),
                           _c_void_p(_ptr(self.error_flag)))
                if partial is not None:
                    # (the leading single tokens are the decode kernel's: their rows stay)
                    skip = singles * heads * splits * (head_dim + 2)
                    self._call("mlxone_attention_merge", _c_void_p(_ptr(partial[skip:])),
                               _c_void_p(_ptr(out[singles:])), _c_int((tokens - singles) * heads),
                               _c_int(splits), _c_int(head_dim))
            else:
                self._call("mlxone_attention_prefill", _c_void_p(_ptr(q)),
                           _c_void_p(_ptr(view.kv)), _c_void_p(_ptr(table)),
                           _c_int(width), _c_int(view.page_size), _c_int(pages),
                           _c_void_p(_ptr(starts)), _c_void_p(_ptr(history)),
                           _c_void_p(_ptr(out)), _c_int(tokens), _c_int(rest),
                           _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_float(scale),
                           _c_int(window or 0))
            return out
        self._call("mlxone_attention_generic", _c_void_p(_ptr(q)), _c_void_p(_ptr(view.kv)),
                   _c_void_p(_ptr(view.block_table)), _c_int(width),
                   _c_int(view.page_size), _c_int(pages),
                   _c_void_p(_ptr(ctx.positions)), _c_void_p(_ptr(ctx.token_request)),
                   _c_void_p(_ptr(out)), _c_int(tokens), _c_int(heads), _c_int(kv_heads),
                   _c_int(head_dim), _c_float(scale), _c_int(window or 0),
                   _c_int(code), _c_void_p(_ptr(self.error_flag)))
        return out

    def _decode_attention(self, q, out, requests, heads, kv_heads, head_dim, scale, window, ctx,
                          view) -> None:
        """The split-key kernel for the first ``requests`` requests of the step, one token each
        (token i is request i's): rows 0 to requests - 1 of q, positions, table and out."""
        width = view.block_table.shape[1]
        splits, partial = self._decode_plan(requests, heads, kv_heads, head_dim, width, window,
                                            view)
        self._call("mlxone_attention_decode", _c_void_p(_ptr(q)), _c_void_p(_ptr(view.kv)),
                   _c_void_p(_ptr(view.block_table)), _c_int(width), _c_int(view.page_size),
                   _c_int(view.kv.shape[1]), _c_void_p(_ptr(ctx.positions)), _c_void_p(_ptr(out)),
                   _c_void_p(_ptr(partial)), _c_int(requests), _c_int(heads), _c_int(kv_heads),
                   _c_int(head_dim), _c_int(splits), _c_float(scale), _c_int(window or 0))
        if partial is not None:
            self.launches += 1          # the merge kernel

    def _decode_plan(self, requests, heads, kv_heads, head_dim, width, window, view):
        """Key splits of a decode attention launch and the scratch for their partial results
        (None when a thread-block cluster merges them, or there is one split)."""
        splits = self.decode_splits(requests, heads, kv_heads, head_dim, width * view.page_size,
                                    window)
        clustered = self.cluster_merge and splits <= min(self.cluster_merge_max_splits, 8)
        partial = None
        if splits > 1 and not clustered:
            partial = torch.empty(requests * heads * splits * (head_dim + 2),
                                  dtype=torch.float32, device=self.device)
        return splits, partial

    def decode_splits(self, requests: int, heads: int, kv_heads: int, head_dim: int,
                      context_bound: int, window: int | None) -> int:
        """Into how many parts the decode kernel cuts a request's keys: as many blocks as the
        GPU holds at once (one wave), but at least four tiles of 32 keys per part."""
        if window:
            context_bound = min(context_bound, window + 31)
        tiles = max(-(-context_bound // 32), 1)
        blocks_per_sm = self.lib.mlxone_attention_decode_resident(_c_int(head_dim))
        groups = kv_heads * (-(-(heads // kv_heads) // 8))
        wanted = max(self._sm_count * blocks_per_sm // max(requests * groups, 1), 1)
        return max(min(wanted, tiles // 4), 1)

    def argmax(self, logits):
        self._need(logits, torch.float32, "logits")
        rows, vocab = logits.shape
        out = torch.empty((rows,), dtype=torch.int32, device=self.device)
        scratch = self.lib.mlxone_argmax_scratch(rows, vocab)
        values = indices = None
        if scratch:
            values = torch.empty(scratch, dtype=torch.float32, device=self.device)
            indices = torch.empty(scratch, dtype=torch.int32, device=self.device)
        self._call("mlxone_argmax", _c_void_p(_ptr(logits)), _c_int(rows), _c_int(vocab),
                   _c_void_p(_ptr(out)), _c_void_p(_ptr(values)), _c_void_p(_ptr(indices)))
        return out

    def decode_advance(self, chosen, token_ids, positions, history, record, counter):
        """In place: token_ids = chosen, positions += 1, history += 1,
        record[counter] = chosen, counter += 1 (all int32 on the device)."""
        for tensor in (chosen, token_ids, positions, history, record, counter):
            self._need(tensor, torch.int32, "decode_advance argument")
        self._call("mlxone_decode_advance", _c_void_p(_ptr(chosen)), _c_void_p(_ptr(token_ids)),
                   _c_void_p(_ptr(positions)), _c_void_p(_ptr(history)), _c_void_p(_ptr(record)),
                   _c_void_p(_ptr(counter)), _c_int(chosen.numel()), _c_int(record.shape[0]))

    def publish_tokens(self, chosen, index, published):
        """published[index[i]] = chosen[i] (all int32 on the device). Returns the step's report
        for the host: the chosen tokens followed by the value of the kernels' error flag, so
        that one copy brings both."""
        report = torch.empty(chosen.numel() + 1, dtype=torch.int32, device=self.device)
        self._call("mlxone_publish_tokens", _c_void_p(_ptr(chosen)), _c_void_p(_ptr(index)),
                   _c_void_p(_ptr(published)), _c_int(chosen.numel()), _c_int(published.numel()),
                   _c_void_p(_ptr(report)), _c_void_p(_ptr(self.error_flag)))
        return report

    def resolve_tokens(self, token_ids, source, published):
        """token_ids[t] = published[source[t]] where source[t] >= 0, in place."""
        self._call("mlxone_resolve_tokens", _c_void_p(_ptr(token_ids)), _c_void_p(_ptr(source)),
                   _c_void_p(_ptr(published)), _c_int(token_ids.numel()),
                   _c_int(published.numel()))

    def reserve_sample_scratch(self, rows: int, vocab: int) -> None:
        """Makes the sampling kernel's scratch large enough for ``rows`` rows now, so that no
        call inside a graph capture has to allocate it."""
        scratch = self._sample_scratch
        if scratch is None or scratch.numel() < rows * vocab:
            self._sample_scratch = torch.empty(rows * vocab, dtype=torch.float32,
                                               device=self.device)

    def sample(self, logits, temperature, top_k, top_p, seed, step):
        """Per row: temperature (float32, > 0), top_k (int32, <= 0 = off), top_p (float32,
        >= 1 = off), seed (int64), step (int32). Returns (tokens int32, probabilities)."""
        self._need(logits, torch.float32, "logits")
        rows, vocab = logits.shape
        for tensor, dtype, what in ((temperature, torch.float32, "temperature"),
                                    (top_k, torch.int32, "top_k"), (top_p, torch.float32, "top_p"),
                                    (seed, torch.int64, "seed"), (step, torch.int32, "step")):
            self._need(tensor, dtype, what)
            if tensor.numel() != rows:
                raise KernelError(f"{what} must have one entry per row")
        scratch = self._sample_scratch
        if scratch is None or scratch.numel() < rows * vocab:
            scratch = torch.empty(rows * vocab, dtype=torch.float32, device=self.device)
            self._sample_scratch = scratch
        out = torch.empty((rows,), dtype=torch.int32, device=self.device)
        self._call("mlxone_sample", _c_void_p(_ptr(logits)), _c_int(rows), _c_int(vocab),
                   _c_void_p(_ptr(temperature)), _c_void_p(_ptr(top_k)), _c_void_p(_ptr(top_p)),
                   _c_void_p(_ptr(seed)), _c_void_p(_ptr(step)), _c_void_p(_ptr(scratch)),
                   _c_void_p(_ptr(out)))
        return out, scratch[: rows * vocab].view(rows, vocab)
