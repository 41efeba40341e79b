"""The Python face of the CUDA kernels: argument checks, output allocation, launches on torch's current stream.

Every method checks what the kernel cannot (device, dtype, contiguity, sizes the kernel refuses)
and raises a clear error instead of launching; a wrong result is never an option. The kernels are
the package's only implementation of these operations: if the library cannot be built or there is
no CUDA device, ``get_kernels`` raises.

Matrix products: in float32 always the package's own CUDA-core kernel (true 32-bit multiply-add in
one fixed order). In bfloat16 the product goes to cuBLAS through ``torch.matmul`` where the
reference's engine also uses the library (its ``nn.Linear`` calls, src/miniserve/model.py:108-111,
160-162,204), except for the 32-bit logits of the output head, which the package's own kernel
produces from bfloat16 inputs with a 32-bit accumulator.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

_DT = {torch.float32: 0, torch.bfloat16: 1}
_ERR_BAD_ARGUMENT = 100001
NUM_SMS_FALLBACK = 148


def _raw_stream(device_index: int) -> int:
    fast = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    return fast(device_index) if fast is not None else torch.cuda.current_stream(device_index).cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


class KernelError(RuntimeError):
    pass


class CudaKernels:
    name = "cuda-sm100a"

    def __init__(self):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: the kernels of this package run on a GPU only")
        self.lib = load_library()
        self.launches = 0
        self.use_cublas = True
        self._attn_scratch: Optional[torch.Tensor] = None
        self._attn_counters: Optional[torch.Tensor] = None
        self._retired: list = []
        self.use_mma_attention = True
        self.sample_single_block = False   # sampling by one block per row instead of a cluster per row (the slower, older kernel)
        self.use_tc_attention = True   # prompt portions of head size 64 or 128: scores and outputs through tcgen05 and tensor memory
        self.cluster_merge = True      # decode attention: the key slices of a token form a cluster and merge in shared memory
        self.use_tc_gemm = True
        self.use_cluster_gate_up = False  # ... by pairs of blocks that share their weight rows (TMA multicast within a cluster of two)
        self.use_pair_gate_up = True     # ... by pairs of multiprocessors on tiles of 256 rows (tcgen05 cta_group::2) ...
        self.pair_gate_up_min_rows = 1024  # ... from this many rows on (measured: 3 to 8 % faster at 2,048 rows, 5 % slower at 512)
        self.use_tc_gate_up = True     # prompt portions: gate/up product with the activation as its epilogue, one tcgen05 kernel
        self.use_tc_qkv = True         # prompt portions, head size 64: q/k/v product with bias, rotation and cache write in one kernel ...
        self.tc_qkv_min_rows = 2048    # ... from this many rows on: below, the library product + the rotation kernel are 4 to 10 % of a step faster
        self.tc_max_rows = 128        # batches up to this many rows take the small-batch tensor-core product
        self.slice_keys = 1024         # generic attention: keys per slice, at fixed places of a request (a multiple of 32)
        self._acc: Optional[torch.Tensor] = None  # float32 zeros: split-K products add into it, their consumer clears it again
        # A library product that is to be added into the residual stream is kept here until the next kernel that reads
        # the stream: that kernel is usually the norm, which adds and normalises in one pass (see ``flush``).
        self._pending_add: Optional[tuple] = None
        self._error_flag: Optional[torch.Tensor] = None
        self._acc_qkv: Optional[torch.Tensor] = None   # float32 sums of a decode step's q/k/v product, read by the attention kernel
        self._dirty_qkv: Optional[torch.Tensor] = None  # those sums while they still wait to be cleared
        self.fuse_decode_rope = True   # decode steps: bias, rotation and cache write happen inside the attention kernel ...
        # ... for heads of 64: 2 to 7 % of a step. The kernel also takes heads of 128, but there it measured 3 % slower at
        # batch 1 and even beyond (a lane then finishes twice as many elements before its first MMA)
        self.fuse_decode_rope_head_dims = (64,)
        self._retired_acc: list = []   # accumulation buffers that were outgrown: captured graphs may still add into and clear them
        self._sms: dict = {}
        self.last_attention_plan = (1, False)   # (key slices, merged as a cluster) of the last tensor-core attention launch
        self._decode_four_warps = False         # the last decode plan asked for blocks of four warps
        for fn in ("llmie_embed", "llmie_feed_tokens", "llmie_zero_fresh_state", "llmie_rope_tables", "llmie_add_rmsnorm", "llmie_rope_kv_write", "llmie_silu_mul",
                   "llmie_gemm_simt", "llmie_gemm_tc", "llmie_gateup_silu_tc", "llmie_qkv_rope_tc", "llmie_add_into", "llmie_attn_plan", "llmie_attn_tc_plan", "llmie_paged_attention_mma", "llmie_paged_attention_mma_acc", "llmie_paged_attention_tc", "llmie_paged_attention_f32", "llmie_paged_attention_bf16", "llmie_argmax", "llmie_sample"):
            getattr(self.lib, fn).restype = ctypes.c_int
        # two forms of the gate/up kernel live in source files of their own, and the library also builds without them
        self._gate_up_cluster = self._gate_up_pair = None
        for attr, name in (("_gate_up_cluster", "llmie_gateup_silu_tc_cluster"), ("_gate_up_pair", "llmie_gateup_silu_tc_pair")):
            try:
                fn = getattr(self.lib, name)
                fn.restype = ctypes.c_int
                setattr(self, attr, fn)
            except AttributeError:
                pass
        # kernels of a step overlap their set-up with the tail of the kernel before (programmatic dependent launch)
        self.lib.llmie_set_pdl(0 if os.environ.get("LLMIE_PDL", "1") == "0" else 1)

    # ------------------------------------------------------------------ helpers
    @property
    def num_sms(self) -> int:
        """Multiprocessors of the device the kernels launch on (torch's current device)."""
        dev = torch.cuda.current_device()
        if dev not in self._sms:
            self._sms[dev] = torch.cuda.get_device_properties(dev).multi_processor_count or NUM_SMS_FALLBACK
        return self._sms[dev]

    def abandon_step(self) -> None:
        """After an exception in the middle of a step: nothing of it may reach the next one. An addition that was put off
        is dropped, and the accumulation buffers, which every product assumes to be zero, are cleared."""
        self._pending_add = None
        self._dirty_qkv = None
        for t in [self._acc, self._acc_qkv, *self._retired_acc]:
            if t is not None:
                try:
                    t.zero_()
                except RuntimeError:
                    pass   # the device itself has failed: nothing more can be done here

    @staticmethod
    def _stream():
        # the raw handle of the current stream, without building a Stream object (this runs before every launch)
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))

    def _check(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc == 0:
            return
        if rc == _ERR_BAD_ARGUMENT:
            raise KernelError(f"{what}: the kernel refused its arguments")
        raise KernelError(f"{what}: CUDA error {rc}")

    @staticmethod
    def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
        if not t.is_cuda:
            raise KernelError(f"{name} must be on a CUDA device")
        if not t.is_contiguous():
            raise KernelError(f"{name} must be contiguous")
        if dtype is not None and t.dtype != dtype:
            raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
        if dims is not None and t.dim() != dims:
            raise KernelError(f"{name} must have {dims} dimensions, got {t.dim()}")

    @staticmethod
    def _dt(t: torch.Tensor, name: str) -> int:
        if t.dtype not in _DT:
            raise KernelError(f"{name} must be float32 or bfloat16, got {t.dtype}")
        return _DT[t.dtype]

    # ------------------------------------------------------------------ kernels
    def embed(self, token_ids, table):
        self._need(token_ids, "token_ids", torch.int32, 1)
        self._need(table, "table", None, 2)
        N, H = token_ids.shape[0], table.shape[1]
        out = torch.empty((N, H), dtype=torch.float32, device=table.device)
        self._check(self.lib.llmie_embed(_ptr(token_ids), _ptr(table), _ptr(out), N, H, self._dt(table, "table"), self._stream()),
                    "embed")
        return out

    def feed_tokens(self, token_ids, source_rows, previous_tokens):
        """``token_ids[i] = previous_tokens[source_rows[i]]`` wherever ``source_rows[i] >= 0`` (all int32, on the device)."""
        for name, t in (("token_ids", token_ids), ("source_rows", source_rows), ("previous_tokens", previous_tokens)):
            self._need(t, name, torch.int32, 1)
        if source_rows.shape[0] != token_ids.shape[0]:
            raise KernelError("feed_tokens: one source row per token is needed")
        self._check(self.lib.llmie_feed_tokens(_ptr(token_ids), _ptr(source_rows), _ptr(previous_tokens), token_ids.shape[0],
                                               self._stream()), "feed_tokens")

    def zero_fresh_state(self, state, seq_slots, seq_starts, positions):
        """``state[seq_slots[r]] = 0`` for every request ``r`` of the step whose rows begin at position 0 (its first portion, or
        a recomputation): fixed-size state of a request starts from zero. Decided on the device: a captured step does it too."""
        self._need(state, "state", torch.float32)
        for name, t in (("seq_slots", seq_slots), ("seq_starts", seq_starts), ("positions", positions)):
            self._need(t, name, torch.int32, 1)
        R = seq_slots.shape[0]
        if seq_starts.shape[0] < R:
            raise KernelError("zero_fresh_state: one start per request is needed")
        if R and state.dim() >= 1 and state.shape[0]:
            self._check(self.lib.llmie_zero_fresh_state(_ptr(state), ctypes.c_longlong(state.numel() // state.shape[0]), _ptr(seq_slots),
                                                        _ptr(seq_starts), _ptr(positions), R, self._stream()), "zero_fresh_state")

    def rope_tables(self, positions, inv_freq):
        self._need(positions, "positions", torch.int32, 1)
        self._need(inv_freq, "inv_freq", torch.float32, 1)
        N, half = positions.shape[0], inv_freq.shape[0]
        cos = torch.empty((N, half), dtype=torch.float32, device=positions.device)
        sin = torch.empty_like(cos)
        self._check(self.lib.llmie_rope_tables(_ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), N, half, self._stream()),
                    "rope_tables")
        return cos, sin

    def _norm(self, residual, delta, weight, eps, rows, out_dtype, what):
        self._need(residual, "residual", torch.float32, 2)
        self._need(weight, "weight", torch.float32, 1)
        H = residual.shape[1]
        if weight.shape[0] != H:
            raise KernelError(f"{what}: weight has {weight.shape[0]} elements, rows have {H}")
        if delta is not None:
            self._need(delta, "delta", out_dtype, 2)
            if delta.shape != residual.shape:
                raise KernelError(f"{what}: delta is {list(delta.shape)}, residual is {list(residual.shape)}")
        if H > 25000:
            raise KernelError(f"{what}: rows of {H} elements do not fit the kernel's shared memory (at most 25000)")
        n_out = residual.shape[0] if rows is None else rows.shape[0]
        if rows is not None:
            self._need(rows, "rows", torch.int32, 1)
        out = torch.empty((n_out, H), dtype=out_dtype, device=residual.device)
        self._check(self.lib.llmie_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), n_out, H,
                                               ctypes.c_float(eps), _DT[out_dtype], self._stream()), what)
        return out

    def flush(self, residual=None) -> None:
        """Carry out an addition into the residual stream that ``linear(add_to=...)`` has put off. Every method of this
        class that reads or writes the stream does this itself; code that reads the stream's tensor directly calls it first."""
        if self._pending_add is None:
            return
        target, y = self._pending_add
        if residual is not None and target.data_ptr() != residual.data_ptr():
            residual = None  # another tensor is wanted: the pending one is finished all the same, nothing may stay behind
        self._pending_add = None
        self._check(self.lib.llmie_add_into(_ptr(target), _ptr(y), target.numel(), self._dt(y, "delta"), self._stream()), "add_into")

    def _take_pending(self, residual, out_dtype):
        """The put-off addend for ``residual`` if there is one that the norm kernel can add on its way (same dtype as its output)."""
        if self._pending_add is None:
            return None
        target, y = self._pending_add
        if target.data_ptr() == residual.data_ptr() and tuple(target.shape) == tuple(residual.shape) and y.dtype == out_dtype:
            self._pending_add = None
            return y
        self.flush()
        return None

    def add_rmsnorm(self, residual, delta, weight, eps, out_dtype):
        if delta is None:
            delta = self._take_pending(residual, out_dtype)
        else:
            self.flush()
        return self._norm(residual, delta, weight, eps, None, out_dtype, "add_rmsnorm")

    def rmsnorm_rows(self, residual, delta, weight, eps, rows, out_dtype):
        self.flush()
        return self._norm(residual, delta, weight, eps, rows, out_dtype, "rmsnorm_rows")

    def _transient(self, M: int, N: int, device) -> torch.Tensor:
        if self._acc is None or self._acc.numel() < M * N or self._acc.device != device:
            if self._acc is not None:
                self._retired_acc.append(self._acc)  # a captured graph may still add into it and clear it: never given back
            self._acc = torch.zeros(max(M * N, 1 << 20), dtype=torch.float32, device=device)
        return self._acc[: M * N].view(M, N)

    def reserve_transient(self, widest: int, device) -> None:
        """Make the accumulation buffer large enough for the small-batch products of a model whose widest projection has
        ``widest`` outputs (a runner does this before anything is captured, so that the buffer need not grow later; if it
        grows all the same, the outgrown buffer is kept for the graphs that hold its address)."""
        self._transient(self.tc_max_rows, widest, torch.device(device))

    def linear(self, x, w, out_dtype=None, add_to=None, transient=False):
        """``x w^T`` for ``x [rows, K]`` and ``w [outputs, K]``.

        ``add_to``: a float32 ``[rows, outputs]`` tensor (the residual stream) that the product is added into;
        nothing is returned. ``transient``: the caller hands the result straight to ``rope_kv_write`` or ``silu_mul``
        and nowhere else; for small bfloat16 batches it is then a float32 view of the library's accumulation buffer,
        which those kernels read and set back to zero."""
        self._need(x, "x", None, 2)
        M, K = x.shape
        N = w.shape[0]
        self._need(w, "w", x.dtype, 2)
        if K != w.shape[1]:
            raise KernelError(f"linear: x has {K} columns, w has {w.shape[1]}")
        bf16 = x.dtype == torch.bfloat16
        small = bf16 and self.use_tc_gemm and M <= self.tc_max_rows and K % 8 == 0
        if add_to is not None:
            self.flush()
            self._need(add_to, "add_to", torch.float32, 2)
            if tuple(add_to.shape) != (M, N):
                raise KernelError(f"linear: add_to is {list(add_to.shape)}, the product is [{M}, {N}]")
            if small:
                self.linear_tc(x, w, out=add_to, accumulate=True)
            elif bf16 and self.use_cublas and add_to.is_contiguous():
                self.launches += 1
                self._pending_add = (add_to, torch.nn.functional.linear(x, w))  # added by the norm that follows, or by flush()
            else:
                self._check(self.lib.llmie_gemm_simt(_ptr(x), _ptr(w), _ptr(add_to), M, N, K, self._dt(x, "x"), 0, 1, self._stream()),
                            "linear (accumulate)")
            return None
        out_dtype = out_dtype or x.dtype
        if small and transient:
            return self.linear_tc(x, w, out=self._transient(M, N, w.device), accumulate=True)
        if small and out_dtype == torch.float32:
            return self.linear_tc(x, w)
        if self.use_cublas and bf16 and out_dtype == torch.bfloat16:
            self.launches += 1
            return torch.nn.functional.linear(x, w)
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        self._check(self.lib.llmie_gemm_simt(_ptr(x), _ptr(w), _ptr(out), M, N, K, self._dt(x, "x"), self._dt(out, "out"), 0,
                                             self._stream()), "linear")
        return out

    def _is_transient(self, t: torch.Tensor) -> bool:
        return self._acc is not None and t.dtype == torch.float32 and t.untyped_storage().data_ptr() == self._acc.untyped_storage().data_ptr()

    def tc_splits(self, M: int, N: int, K: int) -> int:
        """How many blocks share the K range of a small-batch product: enough blocks to draw on the whole memory system
        (three per SM for up to 16 rows, whose blocks are small enough to sit three to an SM; two beyond, as measured), but
        no more atomic additions than the weights are worth."""
        tiles = -(-N // 128) * -(-M // 64)
        nkb = -(-K // 64)
        want = max(1, ((3 if M <= 16 else 2) * self.num_sms) // tiles)
        cap = max(1, (4 << 20) // max(1, M * N))
        return max(1, min(want, nkb, cap))

    def linear_tc(self, x, w, out=None, accumulate=False, k_splits=None):
        """``out (+)= x w^T`` in float32 from bfloat16 operands on the tcgen05 tensor cores, for small batches.
        ``accumulate`` adds into ``out`` (which may be a strided view, e.g. the residual stream) atomically."""
        self._need(w, "w", torch.bfloat16, 2)
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"linear_tc: x has {K} columns, w has {w.shape[1]}")
        if K % 8:
            raise KernelError(f"linear_tc: the inner size {K} must be a multiple of 8 (rows are fetched in 16-byte units)")
        if out is None:
            if accumulate:
                raise KernelError("linear_tc: accumulate needs an output to add into")
            out = torch.empty((M, N), dtype=torch.float32, device=w.device)
        if out.dtype != torch.float32 or out.dim() != 2 or tuple(out.shape) != (M, N) or out.stride(1) != 1:
            raise KernelError("linear_tc: out must be float32 [rows of x, rows of w] with unit column stride")
        self._errors(w.device)
        if k_splits is None:
            k_splits = self.tc_splits(M, N, K) if accumulate else 1
        self._need(x, "x", torch.bfloat16, 2)
        rc = self.lib.llmie_gemm_tc(_ptr(x), _ptr(w), _ptr(out), out.stride(0), M, N, K, int(k_splits), int(bool(accumulate)),
                                    _ptr(self._error_flag), self._stream())
        self._check(rc, "linear_tc")
        return out

    def _errors(self, device) -> torch.Tensor:
        if self._error_flag is None:
            with torch.inference_mode(False):  # an ordinary tensor: it is cleared later from code that runs outside inference mode
                self._error_flag = torch.zeros(1, dtype=torch.int32, device=device)
        return self._error_flag

    def error_flag(self, device) -> torch.Tensor:
        """The device word that a kernel sets when it gives up on a bounded wait (0: nothing happened). Whoever reads a
        step's results back reads this word with them and hands it to ``raise_for_error_code``."""
        return self._errors(torch.device(device))

    def raise_for_error_code(self, code: int) -> None:
        if code:
            if self._error_flag is not None:
                self._error_flag.zero_()
            raise KernelError(f"a block of a tcgen05 kernel gave up waiting on a barrier (code {code}: 1-4 matrix product, "
                              "11-16 attention); its output is not valid, and neither is what later steps made of it")

    def check_device_errors(self) -> None:
        """Raise if a kernel gave up on a bounded wait since the last check (reads one integer back)."""
        if self._error_flag is not None:
            self.raise_for_error_code(int(self._error_flag.item()))

    def rope_kv_write(self, qkv, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size,
                      write_kv=True, out_dtype=None):
        """Bias, rotation and cache write of a fused q/k/v projection; returns the rotated rows in ``out_dtype``
        (the input itself when the types agree). A transient float32 input is consumed and cleared."""
        self._need(qkv, "qkv", None, 2)
        N = qkv.shape[0]
        heads = num_heads + 2 * num_kv_heads
        if qkv.shape[1] != heads * head_dim:
            raise KernelError(f"rope_kv_write: qkv rows have {qkv.shape[1]} elements, the head counts need {heads * head_dim}")
        if head_dim % 2:
            raise KernelError(f"rope_kv_write: head_dim {head_dim} must be even")
        self._need(cos, "cos", torch.float32, 2)
        self._need(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (N, head_dim // 2) or tuple(sin.shape) != (N, head_dim // 2):
            raise KernelError("rope_kv_write: cos and sin must be [tokens, head_dim / 2]")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
            if bias.shape[0] != heads * head_dim:
                raise KernelError("rope_kv_write: bias does not match the projection's width")
        out_dtype = out_dtype or qkv.dtype
        clear = self._is_transient(qkv)
        out = qkv if (out_dtype == qkv.dtype and not clear) else torch.empty(qkv.shape, dtype=out_dtype, device=qkv.device)
        if write_kv:
            self._need(slot_mapping, "slot_mapping", torch.int32, 1)
            for name, pool in (("k_pool", k_pool), ("v_pool", v_pool)):
                self._need(pool, name, out_dtype, 4)
                if tuple(pool.shape[1:]) != (num_kv_heads, page_size, head_dim):
                    raise KernelError(f"rope_kv_write: {name} is {list(pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {head_dim}]")
        self._check(self.lib.llmie_rope_kv_write(_ptr(qkv), _ptr(out), _ptr(bias), _ptr(cos), _ptr(sin), _ptr(slot_mapping), _ptr(k_pool),
                                                 _ptr(v_pool), N, num_heads, num_kv_heads, head_dim, page_size, int(bool(write_kv)),
                                                 int(clear), self._dt(qkv, "qkv"), self._dt(out, "out"), self._stream()), "rope_kv_write")
        return out

    def qkv_rope(self, x, w, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size,
                 write_kv=True, out_dtype=None):
        """The fused q/k/v projection ``x w^T`` with bias, rotation and cache write; returns the rotated rows.

        Prompt portions in bfloat16 with head size 64 take one tcgen05 kernel that does all of it in its epilogue; everything
        else is the product followed by ``rope_kv_write``."""
        out_dtype = out_dtype or x.dtype
        M, K = x.shape
        if (self.use_tc_qkv and x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 and head_dim == 64 and M > self.tc_max_rows
                and M >= self.tc_qkv_min_rows
                and K % 8 == 0 and x.is_contiguous() and w.is_contiguous() and M <= 65535 * 128):
            self._need(w, "w", torch.bfloat16, 2)
            heads = num_heads + 2 * num_kv_heads
            if tuple(w.shape) != (heads * head_dim, K):
                raise KernelError(f"qkv_rope: w is {list(w.shape)}, the head counts and x need [{heads * head_dim}, {K}]")
            self._need(cos, "cos", torch.float32, 2)
            self._need(sin, "sin", torch.float32, 2)
            if tuple(cos.shape) != (M, head_dim // 2) or tuple(sin.shape) != (M, head_dim // 2):
                raise KernelError("qkv_rope: cos and sin must be [tokens, head_dim / 2]")
            if bias is not None:
                self._need(bias, "bias", torch.float32, 1)
                if bias.shape[0] != heads * head_dim:
                    raise KernelError("qkv_rope: bias does not match the projection's width")
            if write_kv:
                self._need(slot_mapping, "slot_mapping", torch.int32, 1)
                for name, pool in (("k_pool", k_pool), ("v_pool", v_pool)):
                    self._need(pool, name, torch.bfloat16, 4)
                    if tuple(pool.shape[1:]) != (num_kv_heads, page_size, head_dim):
                        raise KernelError(f"qkv_rope: {name} is {list(pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {head_dim}]")
            out = torch.empty((M, heads * head_dim), dtype=torch.bfloat16, device=x.device)
            self._check(self.lib.llmie_qkv_rope_tc(_ptr(x), M, K, _ptr(w), _ptr(bias), _ptr(cos), _ptr(sin), _ptr(slot_mapping), _ptr(out),
                                                   _ptr(k_pool), _ptr(v_pool), num_heads, num_kv_heads, head_dim, page_size,
                                                   int(bool(write_kv)), _ptr(self._errors(x.device)), self._stream()), "qkv_rope (tcgen05)")
            return out
        qkv = self.linear(x, w, transient=True)
        return self.rope_kv_write(qkv, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size,
                                  write_kv, out_dtype=out_dtype)

    def attention_slices(self, max_context: int) -> int:
        """Key slices that the generic attention kernel is launched with: slice s of a request always holds its keys
        ``[s * slice_keys, (s + 1) * slice_keys)``, so how a token's keys are cut depends on its own position only, never on
        the batch it is in; a slice beyond a token's position is empty and adds nothing (exactly nothing) to the merge."""
        return max(1, -(-max_context // self.slice_keys))

    def _scratch(self, floats: int, device) -> torch.Tensor:
        if self._attn_scratch is None or self._attn_scratch.numel() < floats or self._attn_scratch.device != device:
            if self._attn_scratch is not None:
                self._retired.append(self._attn_scratch)  # a captured graph may still write there: never given back
            self._attn_scratch = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
        return self._attn_scratch

    def paged_attention(self, qkv, k_pool, v_pool, block_table, token_seq, positions, num_heads, num_kv_heads, head_dim,
                        page_size, scale, window, max_context, batch=None, num_splits=None):
        """Attention of every token of the step over its request's pages. ``batch`` (the step's context, or
        anything with ``seq_lens``, ``seq_starts_dev``, ``max_seq_len`` and a ``_tables`` dict) lets bfloat16
        inputs with head size 64 or 128 take the tensor-core kernels; without it, or for other types and
        sizes, the generic kernel runs."""
        self._need(qkv, "qkv", None, 2)
        dt = self._dt(qkv, "qkv")
        N = qkv.shape[0]
        vec = 4 if dt == 0 else 8
        if head_dim % vec or head_dim > 256:
            raise KernelError(f"paged_attention: head_dim {head_dim} must be a multiple of {vec} and at most 256")
        if num_heads % num_kv_heads:
            raise KernelError("paged_attention: the query heads must be a multiple of the key/value heads")
        if qkv.shape[1] < num_heads * head_dim or qkv.shape[1] % vec:
            raise KernelError("paged_attention: qkv rows are too short for the query heads")
        for name, pool in (("k_pool", k_pool), ("v_pool", v_pool)):
            self._need(pool, name, qkv.dtype, 4)
            if tuple(pool.shape[1:]) != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"paged_attention: {name} is {list(pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {head_dim}]")
        self._need(block_table, "block_table", torch.int32, 2)
        self._need(token_seq, "token_seq", torch.int32, 1)
        self._need(positions, "positions", torch.int32, 1)
        if block_table.shape[1] * page_size < max_context:
            raise KernelError(f"paged_attention: block tables of {block_table.shape[1]} pages cannot hold {max_context} tokens")
        out = torch.empty((N, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        group = num_heads // num_kv_heads
        span = min(max_context, window) if window else max_context
        if (self.use_mma_attention and batch is not None and dt == 1 and head_dim in (64, 128)
                and group <= (16 if batch.max_seq_len == 1 else 64)):
            return self._attention_mma(qkv, k_pool, v_pool, block_table, token_seq, positions, out, num_heads, num_kv_heads,
                                       head_dim, page_size, scale, window, span, batch, num_splits)
        # ``num_splits`` given: that many equal runs of each token's visible keys (tests of the kernel). Otherwise slices at
        # fixed places of the request, which makes the 32-bit path bit-identical however a request is cut into steps
        # and whatever else is in the batch.
        slice_keys = 0 if num_splits else self.slice_keys
        splits = num_splits or self.attention_slices(max_context)
        scratch = self._scratch(N * num_heads * splits * (head_dim + 2), qkv.device) if splits > 1 else None
        fn = self.lib.llmie_paged_attention_f32 if dt == 0 else self.lib.llmie_paged_attention_bf16
        self._check(fn(_ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
                       _ptr(token_seq), _ptr(positions), _ptr(out), _ptr(scratch), N, num_heads, num_kv_heads, head_dim, page_size,
                       ctypes.c_float(scale), int(window), splits, slice_keys, self._stream()), "paged_attention")
        if splits > 1:
            self.launches += 1
        return out

    def _tiles(self, batch, per_tile: int, device):
        """(number of tiles, device table [tiles, 2] of (first token, tokens)) for tiles of up to ``per_tile`` tokens of one request."""
        tiles = sum(-(-n // per_tile) for n in batch.seq_lens)
        key = ("attention tiles", per_tile)
        if key not in batch._tables:
            info = torch.empty((tiles, 2), dtype=torch.int32, device=device)
            self._check(self.lib.llmie_attn_plan(_ptr(batch.seq_starts_dev), len(batch.seq_lens), per_tile, _ptr(info), tiles,
                                                 self._stream()), "attention plan")
            batch._tables[key] = info
        return tiles, batch._tables[key]

    def _attention_tc(self, qkv, k_pool, v_pool, block_table, token_seq, positions, out, num_heads, num_kv_heads, head_dim,
                      page_size, scale, window, span, batch, num_splits):
        """The tcgen05 kernel for prompt portions, if it takes this case: returns ``out`` or None."""
        group = num_heads // num_kv_heads
        if not (self.use_tc_attention and head_dim in (64, 128) and batch.max_seq_len > 1 and group <= 128 and page_size % 8 == 0
                and (64 % page_size == 0 or page_size % 64 == 0) and (num_splits is None or 1 <= num_splits <= 16)):
            return None
        tiles, tile_info = self._tiles(batch, 128 // group, qkv.device)
        if tiles * num_kv_heads > (1 << 20):
            return None
        # A tile's chunks run one after the other, about a microsecond each, and a prompt's last tiles have many times the
        # chunks of its first ones. The plan (made on the device from the step's positions, once per step) cuts the keys of
        # long tiles into slices, as many pieces as fit on the device at once, and starts long pieces first.
        fixed = int(num_splits or 0)
        capacity = max(1, 2 * self.num_sms // num_kv_heads)   # two blocks per SM
        # (tiles of up to 16 chunks are never cut: a slice costs about 8 chunks' time and is at least 8 chunks long)
        max_items = tiles * fixed if fixed else max(tiles, min(capacity, 16 * tiles)) if span > 16 * 64 else tiles
        key = ("tcgen05 attention plan", group, num_kv_heads, page_size, int(window), fixed)
        if key not in batch._tables:
            work = torch.empty((8 * max_items + 4,), dtype=torch.int32, device=qkv.device)
            tmp = torch.empty((3 * tiles,), dtype=torch.int32, device=qkv.device)
            self._check(self.lib.llmie_attn_tc_plan(_ptr(tile_info), tiles, _ptr(positions), _ptr(token_seq), int(window), page_size, capacity, fixed,
                                                    max_items, _ptr(work), _ptr(tmp), self._stream()), "attention plan (tcgen05)")
            batch._tables[key] = (work, tmp)
        work = batch._tables[key][0]
        cells = max_items * num_kv_heads * 128
        buf = self._scratch(cells * (head_dim + 2), qkv.device)
        scratch_o, scratch_ml = buf, buf[cells * head_dim:]
        if self._attn_counters is None or self._attn_counters.device != qkv.device:
            self._attn_counters = torch.zeros(1 << 20, dtype=torch.int32, device=qkv.device)
        self._check(self.lib.llmie_paged_attention_tc(
            _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), ctypes.c_longlong(k_pool.shape[0]), _ptr(block_table),
            block_table.shape[1], tiles, _ptr(work), max_items, _ptr(out),
            _ptr(scratch_o), _ptr(scratch_ml), _ptr(self._attn_counters), num_heads, num_kv_heads, head_dim, page_size,
            ctypes.c_float(scale), int(window), _ptr(self._errors(qkv.device)), self._stream()), "paged_attention (tcgen05)")
        return out

    def _decode_plan(self, tokens, num_kv_heads, head_dim, span, num_splits, device):
        return self._slices(tokens, num_kv_heads, head_dim, span, num_splits, True, device)

    def _slices(self, tiles, num_kv_heads, head_dim, span, num_splits, decode, device):
        """How the tensor-core attention (mma.sync kernels) cuts a tile's keys: (slices, merged as a cluster, scratch for the
        outputs, scratch for maxima and sums, counters)."""
        rows, chunk = (16, 32 if head_dim == 64 else 16) if decode else (64, 64)
        chunks = max(1, -(-span // chunk))
        explicit = num_splits
        if num_splits is None:
            blocks = max(1, tiles * num_kv_heads)
            num_splits = max(1, min(self.num_sms // blocks, chunks // (16 if decode else 8), 64))
            if decode and num_splits > 12:
                # Few requests with long contexts: more slices shorten a block's walk over its keys (its 8 warps take a chunk
                # each, about 0.55 us a round) but lengthen the last block's merge (the slices' partial results come in groups
                # of 12, about a microsecond a trip). Measured at batch 1, context 32768: 64 slices 14.9 us, 32 slices 12.1 us.
                def cost(n):
                    rounds = -(-(-(-chunks // n)) // 8)
                    return rounds * 0.55 + -(-n // 12) * 1.0
                num_splits = min(range(12, num_splits + 1), key=lambda n: (cost(n), -n))
        # Without slices and with more blocks than multiprocessors, blocks of four warps (two per multiprocessor) run in fewer,
        # fuller rounds than blocks of eight (one per multiprocessor) but walk their keys half as fast: what a round costs is a
        # block's start and merge (about 4 us) plus its walk (0.55 us per round of its warps over a chunk each).
        self._decode_four_warps = False
        if decode and num_splits == 1:
            blocks = max(1, tiles * num_kv_heads)
            if blocks > self.num_sms:
                walk = -(-chunks // 8) * 0.55
                self._decode_four_warps = -(-blocks // (2 * self.num_sms)) * (4.0 + 2 * walk) < -(-blocks // self.num_sms) * (4.0 + walk)
        scratch_o = scratch_ml = counters = None
        # Up to four slices of a token merge as one thread-block cluster through shared memory (no trip through global
        # memory); more slices than that go through scratch and a counter: clusters of eight blocks of this size do not
        # all fit on the device at once and were measured slower.
        cluster = int(decode and self.cluster_merge and 1 < num_splits <= (4 if explicit is None else 8))
        self.last_attention_plan = (num_splits, bool(cluster))
        if num_splits > 1 and not cluster:
            cells = tiles * num_kv_heads * num_splits * rows
            buf = self._scratch(cells * (head_dim + 2), device)
            scratch_o, scratch_ml = buf, buf[cells * head_dim:]
            if tiles * num_kv_heads > (1 << 20):
                raise KernelError("paged_attention: too many tiles for the split counters")
            if self._attn_counters is None or self._attn_counters.device != device:
                self._attn_counters = torch.zeros(1 << 20, dtype=torch.int32, device=device)
            counters = self._attn_counters
        return num_splits, cluster, scratch_o, scratch_ml, counters

    def _attention_mma(self, qkv, k_pool, v_pool, block_table, token_seq, positions, out, num_heads, num_kv_heads, head_dim,
                       page_size, scale, window, span, batch, num_splits):
        group = num_heads // num_kv_heads
        decode = batch.max_seq_len == 1
        N = qkv.shape[0]
        if not decode:
            done = self._attention_tc(qkv, k_pool, v_pool, block_table, token_seq, positions, out, num_heads, num_kv_heads, head_dim,
                                      page_size, scale, window, span, batch, num_splits)
            if done is not None:
                return done
        if decode:
            tile_info = None
            num_splits, cluster, scratch_o, scratch_ml, counters = self._decode_plan(N, num_kv_heads, head_dim, span, num_splits, qkv.device)
            tiles = N
        else:
            tiles, tile_info = self._tiles(batch, max(1, 64 // group), qkv.device)
            num_splits, cluster, scratch_o, scratch_ml, counters = self._slices(tiles, num_kv_heads, head_dim, span, num_splits, False, qkv.device)
        self._check(self.lib.llmie_paged_attention_mma(
            _ptr(qkv), qkv.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(token_seq),
            _ptr(positions), _ptr(tile_info), tiles, _ptr(out), _ptr(scratch_o), _ptr(scratch_ml), _ptr(counters), num_heads,
            num_kv_heads, head_dim, page_size, ctypes.c_float(scale), int(window), num_splits,
            2 if (decode and self._decode_four_warps) else int(decode), cluster, self._stream()),
            "paged_attention (tensor cores)")
        return out

    def _clear_dirty(self) -> None:
        """Clear, with a kernel of its own, the projection sums that a fused attention left behind, if no kernel since has done
        it on its way (``silu_mul`` does)."""
        if self._dirty_qkv is not None:
            self._dirty_qkv.zero_()
            self.launches += 1
            self._dirty_qkv = None

    def _qkv_sums(self, rows: int, width: int, device) -> torch.Tensor:
        """Zeroed float32 ``[rows, width]`` that a decode step's q/k/v product adds into and the attention reads. (A buffer of
        its own, not the one ``linear(transient=True)`` hands out: the gate/up product needs that one while this is still dirty.)"""
        need = rows * width
        if self._acc_qkv is None or self._acc_qkv.numel() < need or self._acc_qkv.device != device:
            if self._acc_qkv is not None:
                self._retired_acc.append(self._acc_qkv)
            self._acc_qkv = torch.zeros(max(need, self.tc_max_rows * width), dtype=torch.float32, device=device)
        return self._acc_qkv[:need].view(rows, width)

    def qkv_attention(self, x, w, bias, cos, sin, slot_mapping, k_pool, v_pool, block_table, token_seq, positions, num_heads,
                      num_kv_heads, head_dim, page_size, scale, window, max_context, batch=None, write_kv=True, out_dtype=None):
        """The fused q/k/v projection of the step's rows (bias, rotation, cache write) and their attention over the pages.

        Decode steps in bfloat16 (one row per request, heads of 64, at most 8 query heads per key/value head) take two
        kernels: the small-batch tensor-core product, whose split-K blocks add into float32 sums, and the attention, which
        adds the bias, rotates the queries in its registers and lets the one warp that owns a token's own position finish its
        key and value, put them into its chunk of keys and write them to the cache. Everything else is ``qkv_rope`` followed
        by ``paged_attention``."""
        M, K_ = x.shape
        group = num_heads // max(num_kv_heads, 1)
        width = (num_heads + 2 * num_kv_heads) * head_dim
        if (self.fuse_decode_rope and self.use_mma_attention and self.use_tc_gemm and batch is not None and batch.max_seq_len == 1
                and x.dtype == torch.bfloat16 and (out_dtype or x.dtype) == torch.bfloat16 and head_dim in self.fuse_decode_rope_head_dims and group <= 8
                and num_heads % max(num_kv_heads, 1) == 0 and M <= self.tc_max_rows and K_ % 8 == 0 and tuple(w.shape) == (width, K_)
                and x.is_contiguous() and w.is_contiguous()):
            self._need(cos, "cos", torch.float32, 2)
            self._need(sin, "sin", torch.float32, 2)
            if tuple(cos.shape) != (M, head_dim // 2) or tuple(sin.shape) != (M, head_dim // 2):
                raise KernelError("qkv_attention: cos and sin must be [tokens, head_dim / 2]")
            if bias is not None:
                self._need(bias, "bias", torch.float32, 1)
                if bias.shape[0] != width:
                    raise KernelError("qkv_attention: bias does not match the projection's width")
            for name, pool in (("k_pool", k_pool), ("v_pool", v_pool)):
                self._need(pool, name, torch.bfloat16, 4)
                if tuple(pool.shape[1:]) != (num_kv_heads, page_size, head_dim):
                    raise KernelError(f"qkv_attention: {name} is {list(pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {head_dim}]")
            self._need(block_table, "block_table", torch.int32, 2)
            self._need(token_seq, "token_seq", torch.int32, 1)
            self._need(positions, "positions", torch.int32, 1)
            if write_kv:
                self._need(slot_mapping, "slot_mapping", torch.int32, 1)
            if block_table.shape[1] * page_size < max_context:
                raise KernelError(f"qkv_attention: block tables of {block_table.shape[1]} pages cannot hold {max_context} tokens")
            self._clear_dirty()
            sums = self._qkv_sums(M, width, x.device)
            self.linear_tc(x, w, out=sums, accumulate=True)
            out = torch.empty((M, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
            span = min(max_context, window) if window else max_context
            num_splits, cluster, scratch_o, scratch_ml, counters = self._decode_plan(M, num_kv_heads, head_dim, span, None, x.device)
            self._check(self.lib.llmie_paged_attention_mma_acc(
                _ptr(sums), width, _ptr(bias), _ptr(cos), _ptr(sin), _ptr(slot_mapping if write_kv else None), _ptr(k_pool), _ptr(v_pool),
                _ptr(block_table), block_table.shape[1], _ptr(token_seq), _ptr(positions), M, _ptr(out), _ptr(scratch_o), _ptr(scratch_ml),
                _ptr(counters), num_heads, num_kv_heads, head_dim, page_size, ctypes.c_float(scale), int(window), num_splits, cluster,
                int(self._decode_four_warps), self._stream()), "qkv_attention (tensor cores)")
            self._dirty_qkv = sums
            return out
        qkv = self.qkv_rope(x, w, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size, write_kv,
                            out_dtype=out_dtype)
        return self.paged_attention(qkv, k_pool, v_pool, block_table, token_seq, positions, num_heads, num_kv_heads, head_dim, page_size,
                                    scale, window, max_context, batch=batch)

    def gate_up_act(self, x, w_gate_up, out_dtype=None):
        """``silu(x Wg^T) * (x Wu^T)`` for the fused matrix ``w_gate_up`` ``[2 I, K]`` (gate rows first). Prompt portions in
        bfloat16 take one tcgen05 kernel whose epilogue is the activation (the float32 sums stay in tensor memory; nothing of
        width 2 I is written); everything else is the product followed by ``silu_mul``."""
        out_dtype = out_dtype or x.dtype
        M, K_ = x.shape
        if (self.use_tc_gate_up and x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 and M > self.tc_max_rows and K_ % 8 == 0
                and w_gate_up.dim() == 2 and w_gate_up.shape[0] % 16 == 0 and w_gate_up.shape[1] == K_ and x.is_contiguous()
                and w_gate_up.is_contiguous() and w_gate_up.dtype == torch.bfloat16):
            I = w_gate_up.shape[0] // 2
            out = torch.empty((M, I), dtype=torch.bfloat16, device=x.device)
            # three forms of the kernel: one block per tile of 128 rows; pairs of multiprocessors on tiles of 256 rows
            # (cta_group::2), the default for long portions; pairs of blocks that share their weight rows by TMA multicast,
            # where the library was built with that optional source file (off by default: measured no faster)
            fn = self._gate_up_cluster if (self.use_cluster_gate_up and M > 128) else None
            if self.use_pair_gate_up and self._gate_up_pair is not None and M >= self.pair_gate_up_min_rows:
                fn = self._gate_up_pair
            fn = fn or self.lib.llmie_gateup_silu_tc
            self._check(fn(_ptr(x), _ptr(w_gate_up), _ptr(out), M, I, K_, self.num_sms, _ptr(self._errors(x.device)), self._stream()),
                        "gate_up_act (tcgen05)")
            return out
        return self.silu_mul(self.linear(x, w_gate_up, transient=True), out_dtype)

    def silu_mul(self, gu, out_dtype=None):
        """``silu(gate) * up`` of a fused gate/up projection ``[rows, 2 I]`` (gate first); a transient float32 input is consumed and cleared."""
        self._need(gu, "gate_up", None, 2)
        if gu.shape[1] % 2:
            raise KernelError("silu_mul: the row must hold gate and up halves of equal width")
        N, I = gu.shape[0], gu.shape[1] // 2
        out = torch.empty((N, I), dtype=out_dtype or gu.dtype, device=gu.device)
        # a projection's sums that the attention read but could not clear (several of its blocks read them) are cleared here
        dirty, self._dirty_qkv = self._dirty_qkv, None
        self._check(self.lib.llmie_silu_mul(_ptr(gu), _ptr(out), N, I, int(self._is_transient(gu)), self._dt(gu, "gate_up"),
                                            self._dt(out, "out"), _ptr(dirty), ctypes.c_longlong(0 if dirty is None else dirty.numel()),
                                            self._stream()), "silu_mul")
        return out

    def argmax(self, logits):
        self._need(logits, "logits", torch.float32, 2)
        M, V = logits.shape
        out = torch.empty((M,), dtype=torch.int32, device=logits.device)
        part_v = torch.empty((M * 64,), dtype=torch.float32, device=logits.device)
        part_i = torch.empty((M * 64,), dtype=torch.int32, device=logits.device)
        self._check(self.lib.llmie_argmax(_ptr(logits), _ptr(out), _ptr(part_v), _ptr(part_i), M, V, self._stream()), "argmax")
        self.launches += 1
        return out

    def sample(self, logits, temperature, top_k, top_p, uniform):
        self._need(logits, "logits", torch.float32, 2)
        M, V = logits.shape
        for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                            ("top_p", top_p, torch.float32), ("uniform", uniform, torch.float32)):
            self._need(t, name, dt, 1)
            if t.shape[0] != M:
                raise KernelError(f"sample: {name} needs one value per row")
        out = torch.empty((M,), dtype=torch.int32, device=logits.device)
        self._check(self.lib.llmie_sample(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform), _ptr(out), M, V,
                                          int(self.sample_single_block), self._stream()), "sample")
        return out


_kernels: Optional[CudaKernels] = None


def get_kernels() -> CudaKernels:
    global _kernels
    if _kernels is None:
        _kernels = CudaKernels()
    return _kernels
