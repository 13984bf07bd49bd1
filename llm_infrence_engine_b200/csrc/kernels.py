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
        self.use_fused_router = os.environ.get("LLMIE_FUSED_ROUTER", "1") != "0"   # a router's product and choice in one kernel (few rows, float32)
        self.use_tc_experts = True     # routed experts with many rows per expert: both grouped products on tcgen05 (bfloat16)
        self.use_tc_gate_up = True     # prompt portions: gate/up product with the activation as its epilogue, one tcgen05 kernel
        self.use_tc_qkv = True         # prompt portions, head size 64: q/k/v product with bias, rotation and cache write in one kernel ...
        self.tc_qkv_min_rows = 2048    # ... from this many rows on: below, the library product + the rotation kernel are 4 to 10 % of a step faster
        self.tc_max_rows = 128        # batches up to this many rows take the small-batch tensor-core product
        self.use_mma_attention_ext = True    # bfloat16 attention with extras on the tensor cores (else the generic kernel)
        # ... on tiles of at most this many rows. The kernel also has tiles of 64 and 128 rows (a chunk's keys fetched once for
        # more rows); measured slower at 2,048 tokens (heads of 128: 311 -> 415 us): their registers leave one block per
        # multiprocessor where tiles of 32 rows leave two, and the kernel waits on its barriers, not on the keys
        self.attention_ext_tile_rows = 32
        self.masked_attention_tensor_cores = True    # kept first tokens, chunks and soft caps on the tensor-core kernels too
        self.use_fa_attention_ext = True     # prompt portions with heads of 64 / 128: the kernel in which a warp owns 16 rows and all keys of a chunk
        self.use_mma_attention_talk = True   # heads that talk, steps with prompt portions in bfloat16: plain scores and P V on the tensor cores
        self.head_matmul_library_rows = 64   # per-head products of latent attention: from this many rows on, one batched library product
        self.slice_keys = 1024         # generic attention: keys per slice, at fixed places of a request (a multiple of 32)
        self._acc: Optional[torch.Tensor] = None  # float32 zeros: split-K products add into it, their consumer clears it again
        # A library product that is to be added into the residual stream is kept here until the next kernel that reads
        # the stream: that kernel is usually the norm, which adds and normalises in one pass (see ``flush``).
        self._pending_add: Optional[tuple] = None
        # An update of several residual streams waits here for the norm of the next sublayer, which updates, sums and
        # normalises in one pass: (streams, the sublayer's result, mix, out coefficients)
        self._pending_streams: Optional[tuple] = None
        # A sublayer's result whose layer norm is to be added into the residual stream waits here for the norm of the next
        # sublayer, which adds and normalises in one pass: (stream, result, the post-norm's weight, eps, plain); ``plain``: the result
        # is only scaled element by element by the weight (a layer scale), not normed
        self._pending_post: Optional[tuple] = None
        self._state_lists: dict = {}   # the addresses of a runner's state tensors on the device (zero_fresh_states)
        self._fresh: list = []   # zeroed tensors of ``zeros_like_rows`` that nothing has been added into yet
        # ``zeros_like_rows`` hands out views of one float32 buffer that is zero between uses: the stream kernels that read a
        # sublayer's result out of it set it back to zero on their way (no fill kernel per sublayer)
        self._zero_bufs: list = []
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
                   "llmie_gemm_simt", "llmie_gemm_tc", "llmie_gateup_silu_tc", "llmie_qkv_rope_tc", "llmie_add_into", "llmie_attn_plan", "llmie_attn_tc_plan", "llmie_paged_attention_mma", "llmie_paged_attention_mma_acc", "llmie_paged_attention_tc", "llmie_paged_attention_f32", "llmie_paged_attention_bf16", "llmie_argmax", "llmie_sample",
                   "llmie_streams_expand", "llmie_streams_update", "llmie_streams_norm", "llmie_latent_prepare", "llmie_head_matmul",
                   "llmie_kv_store", "llmie_act", "llmie_paged_attention_ext_f32", "llmie_paged_attention_ext_bf16", "llmie_paged_attention_ext_mma",
                   "llmie_attention_ext_mma_fits", "llmie_paged_attention_ext_fa", "llmie_attention_ext_fa_fits",
                   "llmie_layernorm", "llmie_group_rmsnorm_gate", "llmie_dual_rmsnorm_mix", "llmie_glu_clamped", "llmie_qk_norm_rope_store",
                   "llmie_causal_conv", "llmie_delta_prepare", "llmie_delta_scan", "llmie_ssm_scan", "llmie_zero_fresh_states",
                   "llmie_selective_scan", "llmie_weighted_pair", "llmie_moe_route", "llmie_moe_sort", "llmie_moe_gemm", "llmie_moe_combine",
                   "llmie_moe_tile_rows", "llmie_moe_router", "llmie_moe_gather", "llmie_moe_grouped_tc", "llmie_moe_grouped_tc_rows",
                   "llmie_embed_add", "llmie_mlstm_prepare", "llmie_mlstm_scan", "llmie_mlstm_finish", "llmie_paged_attention_talk",
                   "llmie_attention_talk_slice", "llmie_attention_talk_mma_fits", "llmie_paged_attention_talk_mma"):
            getattr(self.lib, fn).restype = ctypes.c_int
        # two forms of the gate/up kernel live in source files of their own, and the library also builds without them
        self._gate_up_cluster = self._gate_up_pair = self._gate_up_glu_pair = None
        self.lib.llmie_gateup_glu_tc.restype = ctypes.c_int
        for attr, name in (("_gate_up_cluster", "llmie_gateup_silu_tc_cluster"), ("_gate_up_pair", "llmie_gateup_silu_tc_pair"),
                           ("_gate_up_glu_pair", "llmie_gateup_glu_tc_pair")):
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
        self._pending_streams = None
        self._pending_post = None
        self._fresh = []
        self._dirty_qkv = None
        for t in [self._acc, self._acc_qkv, *self._zero_bufs, *self._retired_acc]:
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
    def embed(self, token_ids, table, scale: float = 1.0):
        self._need(token_ids, "token_ids", torch.int32, 1)
        self._need(table, "table", None, 2)
        N, H = token_ids.shape[0], table.shape[1]
        out = torch.empty((N, H), dtype=torch.float32, device=table.device)
        self._check(self.lib.llmie_embed(_ptr(token_ids), _ptr(table), _ptr(out), N, H, self._dt(table, "table"), ctypes.c_float(scale),
                                        self._stream()), "embed")
        return out

    def embed_add(self, token_ids, table, residual, scale: float = 1.0):
        """``residual += table[token] * scale``: the embedding added once more into a stream that already holds something. A sublayer's
        result that still waits to be added stays waiting (additions commute); only a put-off library product is added first."""
        self._need(token_ids, "token_ids", torch.int32, 1)
        self._need(table, "table", None, 2)
        self._need(residual, "residual", torch.float32, 2)
        if tuple(residual.shape) != (token_ids.shape[0], table.shape[1]):
            raise KernelError(f"embed_add: the stream is {list(residual.shape)}, the tokens' rows are [{token_ids.shape[0]}, {table.shape[1]}]")
        if self._pending_add is not None or self._pending_streams is not None:
            self.flush()
        self._check(self.lib.llmie_embed_add(_ptr(token_ids), _ptr(table), _ptr(residual), token_ids.shape[0], table.shape[1], self._dt(table, "table"),
                                            ctypes.c_float(scale), self._stream()), "embed_add")

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

    def zero_fresh_states(self, states, seq_slots, seq_starts, positions):
        """``zero_fresh_state`` for a list of state tensors in one launch (their addresses are put on the device once)."""
        if not states:
            return
        if len(states) == 1:
            return self.zero_fresh_state(states[0], seq_slots, seq_starts, positions)
        key = tuple(t.data_ptr() for t in states)
        if key not in self._state_lists:
            for t in states:
                self._need(t, "state", torch.float32)
            with torch.inference_mode(False):
                ptrs = torch.tensor(key, dtype=torch.int64, device=states[0].device)
                sizes = torch.tensor([t.numel() // t.shape[0] for t in states], dtype=torch.int64, device=states[0].device)
            self._state_lists[key] = (ptrs, sizes)   # (kept for good: a captured step holds their addresses)
        ptrs, sizes = self._state_lists[key]
        for name, t in (("seq_slots", seq_slots), ("seq_starts", seq_starts), ("positions", positions)):
            self._need(t, name, torch.int32, 1)
        R = seq_slots.shape[0]
        if R:
            self._check(self.lib.llmie_zero_fresh_states(_ptr(ptrs), _ptr(sizes), len(states), _ptr(seq_slots),
                                                         _ptr(seq_starts), _ptr(positions), R, self._stream()), "zero_fresh_states")

    def rope_tables(self, positions, inv_freq, mult: float = 1.0):
        self._need(positions, "positions", torch.int32, 1)
        self._need(inv_freq, "inv_freq", torch.float32, 1)
        N, half = positions.shape[0], inv_freq.shape[0]
        cos = torch.empty((N, half), dtype=torch.float32, device=positions.device)
        sin = torch.empty_like(cos)
        self._check(self.lib.llmie_rope_tables(_ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), N, half, ctypes.c_float(mult),
                                              self._stream()), "rope_tables")
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
        if self._pending_add is not None:
            target, y = self._pending_add
            self._pending_add = None
            self._unfresh(target)
            self._check(self.lib.llmie_add_into(_ptr(target), _ptr(y), target.numel(), self._dt(y, "delta"), self._stream()), "add_into")
        if self._pending_streams is not None:
            xs, y, mix, coef_out = self._pending_streams
            self._pending_streams = None
            N, S, H = xs.shape
            self._check(self.lib.llmie_streams_update(_ptr(xs), _ptr(y), self._dt(y, "y"), int(self._clears(y)), _ptr(mix), _ptr(coef_out), N, S, H,
                                                      self._stream()), "streams_update")
        if self._pending_post is not None:
            x, y, w_post, eps, plain = self._pending_post
            self._pending_post = None
            self._layernorm(x, y, w_post, None, eps, None, None, "post_norm_add", post_plain=plain)

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
        which those kernels read and set back to zero. ``x`` may be a run of columns of wider rows (unit column stride): the
        library product takes it as it is, every other path gets a copy."""
        if x.dim() == 2 and not x.is_contiguous():
            as_it_is = (x.stride(1) == 1 and x.dtype == torch.bfloat16 and self.use_cublas and add_to is None and not transient
                        and (out_dtype or x.dtype) == torch.bfloat16 and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0)
            if as_it_is:
                self._need(w, "w", x.dtype, 2)
                if x.shape[1] != w.shape[1]:
                    raise KernelError(f"linear: x has {x.shape[1]} columns, w has {w.shape[1]}")
                self.launches += 1
                return torch.nn.functional.linear(x, w)
            x = x.contiguous()
            self.launches += 1
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
        if bf16 and out_dtype == torch.float32 and self.use_tc_gemm and K % 8 == 0 and N <= 128:
            # few outputs in 32-bit for many rows (a router's logits over a prompt portion): one tile of weight rows, a block per 64 rows
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

    def gate_up_act(self, x, w_gate_up, out_dtype=None, glu=None, activation="silu"):
        """``silu(x Wg^T) * (x Wu^T)`` for the fused matrix ``w_gate_up`` ``[2 I, K]`` (gate rows first). Prompt portions in
        bfloat16 take one tcgen05 kernel whose epilogue is the activation (the float32 sums stay in tensor memory; nothing of
        width 2 I is written); everything else is the product followed by ``silu_mul``. ``glu = (limit, alpha, shift)`` asks for
        the clamped unit ``g sigmoid(alpha g) (u + shift)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)`` instead."""
        out_dtype = out_dtype or x.dtype
        limit, alpha, shift = (float(v) for v in glu) if glu is not None else (0.0, 1.0, 0.0)
        if glu is not None and not limit > 0:
            raise KernelError("gate_up_act: the clamped unit needs a positive limit")
        if activation not in ("silu", "gelu_tanh") or (glu is not None and activation != "silu"):
            raise KernelError(f"gate_up_act: activation '{activation}' is not built")
        if activation == "gelu_tanh":   # ``gelu_tanh(gate) * up``: the kernels of the clamped unit take it as a negative limit
            glu, limit, alpha, shift = (-1.0, 1.0, 0.0), -1.0, 1.0, 0.0
        M, K_ = x.shape
        if (self.use_tc_gate_up and x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 and M > self.tc_max_rows and K_ % 8 == 0
                and w_gate_up.dim() == 2 and w_gate_up.shape[0] % 16 == 0 and w_gate_up.shape[1] == K_ and x.is_contiguous()
                and w_gate_up.is_contiguous() and w_gate_up.dtype == torch.bfloat16):
            I = w_gate_up.shape[0] // 2
            out = torch.empty((M, I), dtype=torch.bfloat16, device=x.device)
            # three forms of the kernel: one block per tile of 128 rows; pairs of multiprocessors on tiles of 256 rows
            # (cta_group::2), the default for long portions; pairs of blocks that share their weight rows by TMA multicast,
            # where the library was built with that optional source file (off by default: measured no faster)
            fn = self._gate_up_cluster if (self.use_cluster_gate_up and M > 128 and glu is None) else None
            pair = self.use_pair_gate_up and self._gate_up_pair is not None and M >= self.pair_gate_up_min_rows
            if pair and glu is None:
                fn = self._gate_up_pair
            if fn is not None or glu is None:
                fn = fn or self.lib.llmie_gateup_silu_tc
                self._check(fn(_ptr(x), _ptr(w_gate_up), _ptr(out), M, I, K_, self.num_sms, _ptr(self._errors(x.device)), self._stream()),
                            "gate_up_act (tcgen05)")
                return out
            fn = self._gate_up_glu_pair if (pair and self._gate_up_glu_pair is not None) else self.lib.llmie_gateup_glu_tc
            self._check(fn(_ptr(x), _ptr(w_gate_up), _ptr(out), M, I, K_, self.num_sms, _ptr(self._errors(x.device)), ctypes.c_float(limit),
                           ctypes.c_float(alpha), ctypes.c_float(shift), self._stream()), "gate_up_act (tcgen05, clamped unit)")
            return out
        if glu is not None:
            return self.glu_clamped(self.linear(x, w_gate_up, transient=True), limit, alpha, shift, out_dtype)
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

    # ------------------------------------------------------------------ several residual streams
    def zeros_like_rows(self, streams, index: int = 0):
        """A zeroed float32 ``[N, hidden]`` for a sublayer to add its result into (``streams`` is ``[N, S, hidden]`` or
        ``[N, hidden]``). ``index`` names one of several such buffers, for a part that needs more than one at a time."""
        N, H = streams.shape[0], streams.shape[-1]
        while len(self._zero_bufs) <= index:
            self._zero_bufs.append(None)
        buf = self._zero_bufs[index]
        if buf is None or buf.numel() < N * H or buf.device != streams.device:
            if buf is not None:
                self._retired_acc.append(buf)   # a captured graph may still add into it and clear it
            with torch.inference_mode(False):   # an ordinary tensor: it is also cleared from code that runs outside inference mode
                buf = self._zero_bufs[index] = torch.zeros(max(N * H, 1 << 20), dtype=torch.float32, device=streams.device)
        out = buf[: N * H].view(N, H)
        self._fresh = [t for t in self._fresh if t.untyped_storage().data_ptr() != buf.untyped_storage().data_ptr()] + [out]
        return out

    def _is_fresh(self, y) -> bool:
        return any(t is y for t in self._fresh)

    def _unfresh(self, y) -> None:
        self._fresh = [t for t in self._fresh if t is not y]

    def _clears(self, y) -> bool:
        return y.dtype == torch.float32 and any(b is not None and y.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()
                                                for b in self._zero_bufs)

    def take_result(self, y):
        """What a sublayer left for a zeroed tensor of ``zeros_like_rows``: the tensor itself (float32 sums), or, where all it
        was to receive is a library product that still waits to be added, that product (and the tensor stays zero)."""
        if self._pending_add is not None and self._pending_add[0] is y and self._is_fresh(y):
            out = self._pending_add[1]
            self._pending_add = None
            self._unfresh(y)
            return out
        self.flush()
        self._unfresh(y)
        return y

    def streams_expand(self, x, streams: int):
        self.flush()
        self._need(x, "x", torch.float32, 2)
        N, H = x.shape
        xs = torch.empty((N, streams, H), dtype=torch.float32, device=x.device)
        self._check(self.lib.llmie_streams_expand(_ptr(x), _ptr(xs), N, streams, H, self._stream()), "streams_expand")
        return xs

    def _check_streams(self, xs, mix, coef_out, what):
        self._need(xs, "streams", torch.float32, 3)
        S = xs.shape[1]
        if S > 16:
            raise KernelError(f"{what}: at most 16 streams, got {S}")
        if mix is not None:
            self._need(mix, "mix", torch.float32, 2)
            self._need(coef_out, "coef_out", torch.float32, 1)
            if tuple(mix.shape) != (S, S) or coef_out.shape[0] != S:
                raise KernelError(f"{what}: mix must be [{S}, {S}] and coef_out [{S}]")

    def streams_update(self, xs, y, mix, coef_out):
        """``xs[:, t] <- sum_s mix[s, t] xs[:, s] + coef_out[t] y``. Put off until the next ``streams_norm`` of the same
        streams (one pass does both) or until ``flush``. If ``y`` is the zeroed tensor of ``zeros_like_rows`` and all it
        holds is a library product that still waits to be added, the product itself is the update and ``y`` is never written."""
        self._check_streams(xs, mix, coef_out, "streams_update")
        y = self.take_result(y)
        self._need(y, "y", None, 2)
        if tuple(y.shape) != (xs.shape[0], xs.shape[2]):
            raise KernelError(f"streams_update: y is {list(y.shape)}, the streams are {list(xs.shape)}")
        self._dt(y, "y")
        self._pending_streams = (xs, y, mix, coef_out)

    def streams_norm(self, xs, coef_in, weight, eps, out_dtype, rows=None):
        """``norm(sum_s coef_in[s] xs[:, s]) * weight`` in ``out_dtype``, of all tokens or of ``rows``; an update of these
        streams that was put off happens in the same kernel (with ``rows`` it is computed for them and not stored)."""
        self._check_streams(xs, None, None, "streams_norm")
        N, S, H = xs.shape
        self._need(coef_in, "coef_in", torch.float32, 1)
        self._need(weight, "weight", torch.float32, 1)
        if coef_in.shape[0] != S or weight.shape[0] != H:
            raise KernelError(f"streams_norm: coef_in must be [{S}] and weight [{H}]")
        y = mix = coef_out = None
        if self._pending_streams is not None and self._pending_streams[0] is xs and self._pending_add is None:
            _, y, mix, coef_out = self._pending_streams
            self._pending_streams = None
        else:
            self.flush()
        if rows is not None:
            self._need(rows, "rows", torch.int32, 1)
        n_out = N if rows is None else rows.shape[0]
        out = torch.empty((n_out, H), dtype=out_dtype, device=xs.device)
        clears = y is not None and self._clears(y)
        self._check(self.lib.llmie_streams_norm(_ptr(xs), _ptr(y), 0 if y is None else self._dt(y, "y"), int(clears), _ptr(mix), _ptr(coef_out),
                                                _ptr(coef_in), _ptr(weight), _ptr(out), _DT[out_dtype], _ptr(rows), n_out, S, H,
                                                ctypes.c_float(eps), self._stream()), "streams_norm")
        if clears and rows is not None:
            y.zero_()   # only the chosen rows were read and cleared; the buffer must be zero for its next user
            self.launches += 1
        return out

    # ------------------------------------------------------------------ a product with an activation behind it
    def linear_act(self, x, w, activation, out_dtype=None):
        """``act(x w^T)``; the activation is computed in 32-bit on the product's sums where those are at hand (small batches)."""
        if activation != "gelu_tanh":
            raise KernelError(f"linear_act: activation '{activation}' is not built")
        out_dtype = out_dtype or x.dtype
        z = self.linear(x, w, transient=True)
        clear = self._is_transient(z)
        out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
        self._check(self.lib.llmie_act(_ptr(z), _ptr(out), ctypes.c_longlong(z.numel()), 0, int(clear), ctypes.c_float(0.0), self._dt(z, "z"),
                                       _DT[out_dtype], self._stream()), "act")
        return out

    def softcap(self, x, cap: float):
        """``cap * tanh(x / cap)`` of a float32 tensor, element by element."""
        self._need(x, "x", torch.float32)
        if not cap > 0:
            raise KernelError("softcap: the cap must be positive")
        out = torch.empty_like(x)
        self._check(self.lib.llmie_act(_ptr(x), _ptr(out), ctypes.c_longlong(x.numel()), 1, 0, ctypes.c_float(cap), 0, 0, self._stream()), "softcap")
        return out

    # ------------------------------------------------------------------ attention with extras
    def kv_store(self, z, k_col, v_col, slot_mapping, k_pool, v_pool, num_kv_heads, head_dim, v_head_dim, page_size):
        """Keys (``num_kv_heads * head_dim`` columns of ``z`` from ``k_col``) and values (from ``v_col``) into the tokens' cache slots."""
        self._need(z, "z", None, 2)
        self._need(slot_mapping, "slot_mapping", torch.int32, 1)
        for name, pool, d in (("k_pool", k_pool, head_dim), ("v_pool", v_pool, v_head_dim)):
            self._need(pool, name, z.dtype, 4)
            if tuple(pool.shape[1:]) != (num_kv_heads, page_size, d):
                raise KernelError(f"kv_store: {name} is {list(pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {d}]")
        if max(k_col + num_kv_heads * head_dim, v_col + num_kv_heads * v_head_dim) > z.shape[1]:
            raise KernelError("kv_store: the key or value columns lie outside the rows")
        self._check(self.lib.llmie_kv_store(_ptr(z), z.shape[1], k_col, v_col, _ptr(slot_mapping), _ptr(k_pool), _ptr(v_pool), z.shape[0],
                                            num_kv_heads, head_dim, v_head_dim, page_size, self._dt(z, "z"), self._stream()), "kv_store")

    def attention_ext(self, q, q_col, num_heads, num_kv_heads, head_dim, v_head_dim, k_pool, v_pool, block_table, token_seq, positions,
                      page_size, scale, window, max_context, temp=(0.0, 0), rel=None, rel_rows=None, sink=None, gate=None, gate_col=0,
                      gate_per_head=False, batch=None, num_splits=None, keep_first=0, chunk=0, softcap=0.0, talk=None):
        """Paged attention with extras: the query heads are columns ``q_col ..`` of ``q``; ``v_pool=None`` reads the values out
        of the key rows (their first ``v_head_dim`` entries); ``temp=(coef, every)`` a query temperature by position;
        ``rel [rows, heads]`` with ``rel_rows`` (distance -> row) a bias by distance; ``sink [heads]`` joins the denominator;
        ``gate`` (columns from ``gate_col`` of a tensor with the tokens' rows) an output gate per head or per element;
        ``keep_first`` keys at the request's start stay visible when the ``window`` has passed them; ``chunk`` > 0 lets a position
        see only the keys of its own run of ``chunk`` positions; ``softcap`` > 0 bounds the scaled scores by ``cap * tanh(s / cap)``;
        ``talk [heads, heads]`` (float32) mixes the heads' capped scores before mask and softmax, ``score'_h = sum_g talk[h, g] score_g``."""
        self._need(q, "q", None, 2)
        dt = self._dt(q, "q")
        N = q.shape[0]
        if num_heads % num_kv_heads:
            raise KernelError("attention_ext: the query heads must be a multiple of the key/value heads")
        if q_col + num_heads * head_dim > q.shape[1]:
            raise KernelError("attention_ext: the rows are too short for the query heads")
        self._need(k_pool, "k_pool", q.dtype, 4)
        if tuple(k_pool.shape[1:]) != (num_kv_heads, page_size, head_dim):
            raise KernelError(f"attention_ext: k_pool is {list(k_pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {head_dim}]")
        if v_pool is not None:
            self._need(v_pool, "v_pool", q.dtype, 4)
            if tuple(v_pool.shape[1:]) != (num_kv_heads, page_size, v_head_dim):
                raise KernelError(f"attention_ext: v_pool is {list(v_pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {v_head_dim}]")
        elif v_head_dim > head_dim:
            raise KernelError("attention_ext: values read out of the key rows cannot be longer than the keys")
        self._need(block_table, "block_table", torch.int32, 2)
        self._need(token_seq, "token_seq", torch.int32, 1)
        self._need(positions, "positions", torch.int32, 1)
        if block_table.shape[1] * page_size < max_context:
            raise KernelError(f"attention_ext: block tables of {block_table.shape[1]} pages cannot hold {max_context} tokens")
        if rel is not None:
            self._need(rel, "rel", torch.float32, 2)
            self._need(rel_rows, "rel_rows", torch.int32, 1)
            if rel.shape[1] != num_heads:
                raise KernelError("attention_ext: rel needs one column per head")
        if sink is not None:
            self._need(sink, "sink", torch.float32, 1)
            if sink.shape[0] != num_heads:
                raise KernelError("attention_ext: sink needs one number per head")
        gate_mode = 0
        if gate is not None:
            self._need(gate, "gate", q.dtype, 2)
            gate_mode = 1 if gate_per_head else 2
            if gate.shape[0] != N or gate_col + (num_heads if gate_per_head else num_heads * v_head_dim) > gate.shape[1]:
                raise KernelError("attention_ext: the gate columns lie outside the rows")
        out = torch.empty((N, num_heads * v_head_dim), dtype=q.dtype, device=q.device)
        esize = q.element_size()
        if talk is not None:
            return self._attention_talk(q, q_col, num_heads, num_kv_heads, head_dim, v_head_dim, k_pool, v_pool, block_table, token_seq, positions,
                                        page_size, scale, window, max_context, talk, sink, gate, gate_col, gate_mode, keep_first, chunk, softcap,
                                        temp, rel, out, batch)
        max_rows = 0
        tensor_cores = dt == 1 and self.use_mma_attention_ext and batch is not None and (q_col * esize) % 16 == 0 and q.shape[1] % 8 == 0
        masked = bool(keep_first or chunk or softcap)
        if masked and not self.masked_attention_tensor_cores:
            tensor_cores = False
        if keep_first < 0 or chunk < 0 or softcap < 0 or (keep_first and not window):
            raise KernelError("attention_ext: keep_first needs a window, and keep_first, chunk and softcap cannot be negative")
        if (tensor_cores and self.use_fa_attention_ext and batch.max_seq_len > 1
                and self.lib.llmie_attention_ext_fa_fits(head_dim, v_head_dim, int(v_pool is not None), num_heads // num_kv_heads)):
            # steps with prompt portions, heads of 64 or 128: tiles of 64 rows, a warp to 16 rows and all of a chunk's keys
            group = num_heads // num_kv_heads
            tiles, tile_info = self._tiles(batch, 64 // min(group, 64), q.device)
            blocks = tiles * num_kv_heads * -(-group // 64)
            span = min(max_context, window, chunk or max_context) if window else min(max_context, chunk or max_context)
            splits = num_splits or max(1, min((2 * self.num_sms) // max(blocks, 1), -(-span // 64) // 2, 32))
            scratch = self._scratch(N * num_heads * splits * (v_head_dim + 2), q.device) if splits > 1 else None
            self._check(self.lib.llmie_paged_attention_ext_fa(
                ctypes.c_void_p(q.data_ptr() + q_col * esize), q.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
                _ptr(token_seq), _ptr(positions), _ptr(tile_info), tiles, _ptr(out), _ptr(scratch), N, num_heads, num_kv_heads, head_dim,
                v_head_dim, page_size, ctypes.c_float(scale), int(window), splits, ctypes.c_float(temp[0]), int(temp[1]), _ptr(rel),
                _ptr(rel_rows), 0 if rel_rows is None else rel_rows.shape[0], 0 if rel is None else rel.shape[0], _ptr(sink),
                ctypes.c_void_p(0 if gate is None else gate.data_ptr() + gate_col * esize), 0 if gate is None else gate.shape[1], gate_mode,
                int(keep_first), int(chunk), ctypes.c_float(softcap), self._stream()), "attention_ext (tensor cores, a warp to a row block)")
            if splits > 1:
                self.launches += 1
            return out
        if tensor_cores:
            max_rows = self.lib.llmie_attention_ext_mma_fits(head_dim, v_head_dim, int(v_pool is not None))
        if max_rows:
            # bfloat16: the tensor-core kernel, for prompt portions and decoded tokens alike. A tile is 32, 64 or 128 rows of
            # (token, head of the group), as many as the step's longest request can fill; the keys are cut into slices when
            # the tiles alone would leave multiprocessors idle.
            group = num_heads // num_kv_heads
            heads_per_tile = min(group, 32)
            tile_rows = 32
            while tile_rows < min(max_rows, self.attention_ext_tile_rows) and tile_rows < batch.max_seq_len * heads_per_tile:
                tile_rows *= 2
            if batch.max_seq_len == 1:
                tiles, tile_info = N, None
            else:
                tiles, tile_info = self._tiles(batch, tile_rows // heads_per_tile, q.device)
            blocks = tiles * num_kv_heads * -(-group // heads_per_tile)
            span = min(max_context, window, chunk or max_context) if window else min(max_context, chunk or max_context)
            splits = num_splits or max(1, min((2 * self.num_sms) // max(blocks, 1), -(-span // 64) // 2, 32))
            scratch = self._scratch(N * num_heads * splits * (v_head_dim + 2), q.device) if splits > 1 else None
            self._check(self.lib.llmie_paged_attention_ext_mma(
                ctypes.c_void_p(q.data_ptr() + q_col * esize), q.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
                _ptr(token_seq), _ptr(positions), _ptr(tile_info), tiles, tile_rows, _ptr(out), _ptr(scratch), N, num_heads, num_kv_heads,
                head_dim, v_head_dim, page_size, ctypes.c_float(scale), int(window), splits, ctypes.c_float(temp[0]), int(temp[1]), _ptr(rel),
                _ptr(rel_rows), 0 if rel_rows is None else rel_rows.shape[0], 0 if rel is None else rel.shape[0], _ptr(sink),
                ctypes.c_void_p(0 if gate is None else gate.data_ptr() + gate_col * esize), 0 if gate is None else gate.shape[1], gate_mode,
                int(keep_first), int(chunk), ctypes.c_float(softcap), self._stream()), "attention_ext (tensor cores)")
            if splits > 1:
                self.launches += 1
            return out
        slice_keys = 0 if num_splits else self.slice_keys
        splits = num_splits or self.attention_slices(max_context)
        scratch = self._scratch(N * num_heads * splits * (v_head_dim + 2), q.device) if splits > 1 else None
        fn = self.lib.llmie_paged_attention_ext_f32 if dt == 0 else self.lib.llmie_paged_attention_ext_bf16
        self._check(fn(ctypes.c_void_p(q.data_ptr() + q_col * esize), q.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                       block_table.shape[1], _ptr(token_seq), _ptr(positions), _ptr(out), _ptr(scratch), N, num_heads, num_kv_heads,
                       head_dim, v_head_dim, page_size, ctypes.c_float(scale), int(window), splits, slice_keys,
                       ctypes.c_float(temp[0]), int(temp[1]), _ptr(rel), _ptr(rel_rows), 0 if rel_rows is None else rel_rows.shape[0],
                       0 if rel is None else rel.shape[0], _ptr(sink),
                       ctypes.c_void_p(0 if gate is None else gate.data_ptr() + gate_col * esize), 0 if gate is None else gate.shape[1],
                       gate_mode, int(keep_first), int(chunk), ctypes.c_float(softcap), self._stream()), "attention_ext")
        if splits > 1:
            self.launches += 1
        return out

    def _attention_talk(self, q, q_col, num_heads, num_kv_heads, head_dim, v_head_dim, k_pool, v_pool, block_table, token_seq, positions, page_size,
                        scale, window, max_context, talk, sink, gate, gate_col, gate_mode, keep_first, chunk, softcap, temp, rel, out, batch):
        """Attention whose heads' scores are mixed before the softmax: one block serves all heads of a token and a slice of its keys. The
        slices lie at fixed places of a request (as many keys as fit the shared memory with all heads' scores), so a token's result
        depends on its own position alone."""
        self._need(talk, "talk", torch.float32, 2)
        if tuple(talk.shape) != (num_heads, num_heads):
            raise KernelError(f"attention_ext: talk must be [{num_heads}, {num_heads}]")
        if rel is not None or temp[1]:
            raise KernelError("attention_ext: talking heads are not built together with a bias by distance or a query temperature")
        N = q.shape[0]
        esize = q.element_size()
        per_tile = 0
        if (self.use_mma_attention_talk and q.dtype == torch.bfloat16 and batch is not None and batch.max_seq_len > 1 and v_pool is not None
                and not (window or keep_first or chunk) and gate_mode != 2 and (q_col * esize) % 16 == 0 and q.shape[1] % 8 == 0):
            per_tile = self.lib.llmie_attention_talk_mma_fits(num_heads, num_kv_heads, head_dim, v_head_dim)
        if per_tile:
            # steps with prompt portions, bfloat16: a tile of 16 / (heads per key/value head) tokens and all heads on the tensor cores
            tiles, tile_info = self._tiles(batch, per_tile, q.device)
            self._check(self.lib.llmie_paged_attention_talk_mma(
                ctypes.c_void_p(q.data_ptr() + q_col * esize), q.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
                _ptr(token_seq), _ptr(positions), _ptr(tile_info), tiles, _ptr(talk), _ptr(out), num_heads, num_kv_heads, head_dim, v_head_dim,
                page_size, ctypes.c_float(scale), _ptr(sink), ctypes.c_void_p(0 if gate is None else gate.data_ptr() + gate_col * esize),
                0 if gate is None else gate.shape[1], ctypes.c_float(softcap), self._stream()), "attention_ext (talking heads, tensor cores)")
            return out
        slice_keys = self.lib.llmie_attention_talk_slice(num_heads, head_dim)
        if slice_keys < 32:
            raise KernelError(f"attention_ext: {num_heads} talking heads of {head_dim} entries do not fit the kernel's shared memory")
        splits = max(1, -(-max_context // slice_keys))
        scratch = self._scratch(N * num_heads * splits * (v_head_dim + 2), q.device) if splits > 1 else None
        self._check(self.lib.llmie_paged_attention_talk(
            ctypes.c_void_p(q.data_ptr() + q_col * esize), q.shape[1], _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
            _ptr(token_seq), _ptr(positions), _ptr(talk), _ptr(out), _ptr(scratch), N, num_heads, num_kv_heads, head_dim, v_head_dim, page_size,
            ctypes.c_float(scale), int(window), splits, slice_keys, _ptr(sink),
            ctypes.c_void_p(0 if gate is None else gate.data_ptr() + gate_col * esize), 0 if gate is None else gate.shape[1], gate_mode,
            int(keep_first), int(chunk), ctypes.c_float(softcap), self._dt(q, "q"), self._stream()), "attention_ext (talking heads)")
        if splits > 1:
            self.launches += 1
        return out

    # ------------------------------------------------------------------ the matrix memory with exponential gates
    def mlstm(self, z, q_col, k_col, v_col, gates, bias_i, bias_f, cap, num_heads, head_dim, v_head_dim, state, mstate, batch):
        """The mLSTM recurrence over the rows of each request. ``z`` holds q, k (``heads * head_dim`` columns from ``q_col``, ``k_col``) and v
        (``heads * v_head_dim`` from ``v_col``); ``gates [N, >= 2 heads]`` float32 are the pre-activations ``[W_i h | W_f h]`` of the two
        gates. With ``i = cap tanh((x_i + b_i) / cap)`` and ``f = ln sigmoid(cap tanh((x_f + b_f) / cap))`` (``cap`` None: no cap), per head:
        ``m <- max(f + m, i)``; ``S <- exp(f + m_old - m) S + exp(i - m) k v^T``, ``n`` likewise with ``k`` alone. From ``state [slots, heads,
        v_head_dim + 1, head_dim]`` (the memory column by column, the normaliser as its last column) and ``mstate [slots, heads]``, which
        are moved on. Returns the numerators ``[N, heads, v_head_dim + 1]`` (``S^T q`` with ``q`` times ``head_dim^-1/2``, then ``n . q``)
        and ``m [N, heads]``, float32: ``mlstm_finish`` divides, norms and gates."""
        self._need(z, "z", None, 2)
        self._need(gates, "gates", torch.float32, 2)
        self._need(state, "state", torch.float32, 4)
        self._need(mstate, "mstate", torch.float32, 2)
        self._need(bias_i, "bias_i", torch.float32, 1)
        self._need(bias_f, "bias_f", torch.float32, 1)
        N, H, D, DV = z.shape[0], num_heads, head_dim, v_head_dim
        if max(q_col, k_col) + H * D > z.shape[1] or v_col + H * DV > z.shape[1] or gates.shape[0] != N or gates.shape[1] < 2 * H:
            raise KernelError("mlstm: the columns of q, k, v or the gates lie outside the rows")
        if tuple(state.shape[1:]) != (H, DV + 1, D) or tuple(mstate.shape[1:]) != (H,) or mstate.shape[0] != state.shape[0]:
            raise KernelError(f"mlstm: state is {list(state.shape)} / {list(mstate.shape)}, expected [slots, {H}, {DV + 1}, {D}] / [slots, {H}]")
        if bias_i.shape[0] != H or bias_f.shape[0] != H:
            raise KernelError("mlstm: one bias per head and gate is needed")
        if D > 256:
            raise KernelError(f"mlstm: head_dim {D} is more than the 256 entries of a column that the kernel keeps in registers")
        dev = z.device
        work = torch.empty((2 * N * H * D + 2 * N * H,), dtype=torch.float32, device=dev)
        qf, kf = work[:N * H * D], work[N * H * D:2 * N * H * D]
        ig, fg = work[2 * N * H * D:2 * N * H * D + N * H], work[2 * N * H * D + N * H:]
        dt = self._dt(z, "z")
        self._check(self.lib.llmie_mlstm_prepare(_ptr(z), z.shape[1], q_col, k_col, _ptr(gates), gates.shape[1], _ptr(bias_i), _ptr(bias_f),
                                                 ctypes.c_float(cap or 0.0), ctypes.c_float(D ** -0.5), _ptr(qf), _ptr(kf), _ptr(ig), _ptr(fg), N, H, D, dt,
                                                 self._stream()), "mlstm (prepare)")
        num = torch.empty((N, H, DV + 1), dtype=torch.float32, device=dev)
        m = torch.empty((N, H), dtype=torch.float32, device=dev)
        self._check(self.lib.llmie_mlstm_scan(_ptr(z), z.shape[1], v_col, _ptr(qf), _ptr(kf), _ptr(ig), _ptr(fg), _ptr(state), _ptr(mstate),
                                              _ptr(batch.seq_starts_dev), _ptr(batch.seq_slots), _ptr(num), _ptr(m), H, D, DV, batch.num_seqs, dt,
                                              self._stream()), "mlstm (scan)")
        return num, m

    def mlstm_finish(self, num, m, gate, gate_col, weight, eps, out_dtype):
        """``o = num[..., :DV] / (max(|num[..., DV]|, exp(-m)) + 1e-6)``; every head's ``o`` divided by its root mean square, times
        ``weight [heads * DV]``, times ``sigmoid`` of the gate columns (``heads * DV`` from ``gate_col`` of ``gate``); ``[N, heads * DV]``."""
        self._need(num, "num", torch.float32, 3)
        self._need(m, "m", torch.float32, 2)
        self._need(gate, "gate", out_dtype, 2)
        self._need(weight, "weight", torch.float32, 1)
        N, H, DV = num.shape[0], num.shape[1], num.shape[2] - 1
        if tuple(m.shape) != (N, H) or weight.shape[0] != H * DV or gate.shape[0] != N or gate_col + H * DV > gate.shape[1]:
            raise KernelError("mlstm_finish: the maxima, the weight or the gate columns do not fit the numerators")
        out = torch.empty((N, H * DV), dtype=out_dtype, device=num.device)
        self._check(self.lib.llmie_mlstm_finish(_ptr(num), _ptr(m), ctypes.c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1],
                                                _ptr(weight), _ptr(out), N, H, DV, ctypes.c_float(eps), _DT[out_dtype], self._stream()), "mlstm_finish")
        return out

    # ------------------------------------------------------------------ layer norm before and after a sublayer
    def _layernorm(self, x, y, w_post, w_pre, eps, rows, out_dtype, what, b_pre=None, post_plain=False):
        self._need(x, "residual", torch.float32, 2)
        N, H = x.shape
        clear = False
        y_dt = 0
        if y is not None:
            self._need(y, "y", None, 2)
            y_dt = self._dt(y, "y")
            if tuple(y.shape) != (N, H):
                raise KernelError(f"{what}: the sublayer's result is {list(y.shape)}, the stream is {list(x.shape)}")
            self._need(w_post, "w_post", torch.float32, 1)
            if w_post.shape[0] != H:
                raise KernelError(f"{what}: the post-norm's weight has {w_post.shape[0]} elements, rows have {H}")
            clear = self._clears(y)
        if H > 12500:
            raise KernelError(f"{what}: rows of {H} elements do not fit the kernel's shared memory (at most 12500)")
        out = None
        out_dt = y_dt
        n_out = N if rows is None else rows.shape[0]
        if rows is not None:
            self._need(rows, "rows", torch.int32, 1)
        if w_pre is not None:
            self._need(w_pre, "weight", torch.float32, 1)
            if w_pre.shape[0] != H:
                raise KernelError(f"{what}: weight has {w_pre.shape[0]} elements, rows have {H}")
            if b_pre is not None:
                self._need(b_pre, "bias", torch.float32, 1)
                if b_pre.shape[0] != H:
                    raise KernelError(f"{what}: bias has {b_pre.shape[0]} elements, rows have {H}")
            out = torch.empty((n_out, H), dtype=out_dtype, device=x.device)
            out_dt = _DT[out_dtype]
            if y is None:
                y_dt = 0
            elif y_dt == 1 and out_dt == 0:
                raise KernelError(f"{what}: a rounded result cannot feed a float32 norm")
        elif y is None:
            return None
        self._check(self.lib.llmie_layernorm(_ptr(x), _ptr(y), y_dt, _ptr(w_post), int(clear), _ptr(w_pre), _ptr(b_pre if w_pre is not None else None), _ptr(out), out_dt, _ptr(rows), n_out, H,
                                             ctypes.c_float(eps), int(bool(post_plain)), self._stream()), what)
        if clear and rows is not None:
            y.zero_()   # only the chosen rows were read and cleared; the buffer must be zero for its next user
            self.launches += 1
        return out

    def layernorm(self, residual, weight, eps, out_dtype, rows=None, bias=None):
        """``(x - mean) / sqrt(var + eps) * weight (+ bias)`` of the stream's rows (or of ``rows``), in ``out_dtype``. A sublayer's result
        whose own layer norm still waits to be added into this stream (``post_norm_add``) is added by the same kernel."""
        y = w_post = None
        plain = False
        if (self._pending_post is not None and self._pending_post[0] is residual and (self._pending_post[3] == eps or self._pending_post[4])
                and self._pending_add is None and self._pending_streams is None):
            _, y, w_post, _, plain = self._pending_post
            if y.dtype == torch.bfloat16 and out_dtype == torch.float32:   # no kernel for this pair: the addition on its own, then the norm
                y = w_post = None
                plain = False
                self.flush()
            else:
                self._pending_post = None
        else:
            self.flush()
        return self._layernorm(residual, y, w_post, weight, eps, rows, out_dtype, "layernorm", b_pre=bias, post_plain=plain)

    def post_norm_add(self, residual, y, weight, eps):
        """``residual += layernorm(y) * weight``: put off until the next ``layernorm`` of the same stream (one pass does both)
        or until ``flush``. ``y`` is a zeroed tensor of ``zeros_like_rows`` that the sublayer added its result into."""
        y = self.take_result(y)
        self._pending_post = (residual, y, weight, float(eps), False)

    def scaled_add(self, residual, y, weight):
        """``residual += y * weight`` element by element (a layer scale on a sublayer's result): put off until the next ``layernorm``
        of the same stream (one pass does both) or until ``flush``. ``y`` is a zeroed tensor of ``zeros_like_rows`` that the sublayer
        added its result into."""
        y = self.take_result(y)
        self._need(weight, "weight", torch.float32, 1)
        self._pending_post = (residual, y, weight, 0.0, True)

    def group_rmsnorm_gate(self, x, gate, gate_col, weight, group_size, eps, gate_first, out_dtype, gate_act="sigmoid"):
        """Float32 rows ``x [N, C]`` normed by their root mean square in groups of ``group_size`` channels, with a gate read
        from columns ``gate_col ..`` of ``gate``: ``gate_first`` multiplies by ``silu(gate)`` before the norm, otherwise by
        ``sigmoid(gate)`` (or, with ``gate_act="silu"``, by ``silu(gate)``) after it. ``weight`` has one entry per channel, or one
        per channel of a group (shared by all groups)."""
        if gate_act not in ("sigmoid", "silu") or (gate_first and gate_act != "sigmoid"):
            raise KernelError("group_rmsnorm_gate: the gate after the norm is 'sigmoid' or 'silu'; before the norm it is always silu")
        self._need(x, "x", torch.float32, 2)
        N, C = x.shape
        self._need(weight, "weight", torch.float32, 1)
        if gate.dim() != 2 or gate.stride(1) != 1 or gate.shape[0] != N or gate_col + C > gate.shape[1] or gate.dtype != out_dtype:
            raise KernelError("group_rmsnorm_gate: the gate must be rows of the output's type that hold a column for every channel")
        if C % group_size or weight.shape[0] not in (C, group_size):
            raise KernelError("group_rmsnorm_gate: the groups or the weight do not fit the channels")
        out = torch.empty((N, C), dtype=out_dtype, device=x.device)
        self._check(self.lib.llmie_group_rmsnorm_gate(_ptr(x), ctypes.c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.stride(0),
                                                      self._dt(gate, "gate"), _ptr(weight), weight.shape[0], _ptr(out), _DT[out_dtype], N, C,
                                                      group_size, ctypes.c_float(eps), 0 if gate_first else (2 if gate_act == "silu" else 1), self._stream()), "group_rmsnorm_gate")
        return out

    def dual_rmsnorm_mix(self, a, b, weight_a, weight_b, eps, coef, add_to):
        """``add_to += coef * (a / rms(a) * weight_a + b / rms(b) * weight_b)`` row by row (``add_to`` float32)."""
        self.flush()
        self._need(add_to, "add_to", torch.float32, 2)
        N, H = add_to.shape
        for name, t in (("a", a), ("b", b)):
            self._need(t, name, None, 2)
            if tuple(t.shape) != (N, H):
                raise KernelError(f"dual_rmsnorm_mix: {name} is {list(t.shape)}, the target is {list(add_to.shape)}")
        self._need(weight_a, "weight_a", torch.float32, 1)
        self._need(weight_b, "weight_b", torch.float32, 1)
        self._check(self.lib.llmie_dual_rmsnorm_mix(_ptr(a), self._dt(a, "a"), _ptr(b), self._dt(b, "b"), _ptr(weight_a), _ptr(weight_b), _ptr(add_to),
                                                    N, H, ctypes.c_float(eps), ctypes.c_float(coef), 1, int(self._clears(a)), int(self._clears(b)), self._stream()),
                    "dual_rmsnorm_mix")
        self._unfresh(add_to)

    def weighted_pair(self, a, b, coef_a, coef_b, add_to):
        """``add_to += coef_a * a + coef_b * b`` (``add_to`` float32): two sublayer results of one input, each with its factor."""
        self.flush()
        self._need(add_to, "add_to", torch.float32, 2)
        for name, t in (("a", a), ("b", b)):
            self._need(t, name, None, 2)
            if tuple(t.shape) != tuple(add_to.shape):
                raise KernelError(f"weighted_pair: {name} is {list(t.shape)}, the target is {list(add_to.shape)}")
        self._check(self.lib.llmie_weighted_pair(_ptr(a), self._dt(a, "a"), _ptr(b), self._dt(b, "b"), ctypes.c_float(coef_a), ctypes.c_float(coef_b),
                                                 _ptr(add_to), ctypes.c_longlong(add_to.numel()), int(self._clears(a)), int(self._clears(b)),
                                                 self._stream()), "weighted_pair")
        self._unfresh(add_to)

    def glu_clamped(self, gu, limit, alpha, shift, out_dtype=None):
        """``g * sigmoid(alpha g) * (u + shift)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)`` of a fused gate/up
        projection ``[rows, 2 I]`` (gate first); a transient float32 input is consumed and cleared. A negative ``limit`` asks for
        ``gelu_tanh(gate) * up`` instead."""
        self._need(gu, "gate_up", None, 2)
        if gu.shape[1] % 2:
            raise KernelError("glu_clamped: the row must hold gate and up halves of equal width")
        N, I = gu.shape[0], gu.shape[1] // 2
        out = torch.empty((N, I), dtype=out_dtype or gu.dtype, device=gu.device)
        self._check(self.lib.llmie_glu_clamped(_ptr(gu), _ptr(out), N, I, int(self._is_transient(gu)), ctypes.c_float(limit), ctypes.c_float(alpha),
                                               ctypes.c_float(shift), self._dt(gu, "gate_up"), self._dt(out, "out"), self._stream()), "glu_clamped")
        return out

    # ------------------------------------------------------------------ heads normed and partly rotated on their way to the cache
    def qk_norm_rope_store(self, z, num_heads, num_kv_heads, head_dim, v_head_dim, q_weight, k_weight, eps, cos, sin, rot_dims, interleaved,
                           slot_mapping, k_pool, v_pool, page_size, write_kv=True):
        """From rows ``z = [query heads | key heads | value heads]``: per query and key head an optional RMS norm with a weight,
        then the rotation of its first ``rot_dims`` entries (pairs ``(i, i + rot_dims/2)``, or neighbours when ``interleaved``);
        returns the query heads ``[N, heads * head_dim]`` and puts keys and values into the tokens' cache slots."""
        self._need(z, "z", None, 2)
        N = z.shape[0]
        if z.shape[1] < (num_heads + num_kv_heads) * head_dim + num_kv_heads * v_head_dim:
            raise KernelError("qk_norm_rope_store: the rows are too short for the heads")
        if rot_dims:
            self._need(cos, "cos", torch.float32, 2)
            self._need(sin, "sin", torch.float32, 2)
            if rot_dims % 2 or rot_dims > head_dim or tuple(cos.shape) != (N, rot_dims // 2) or tuple(sin.shape) != (N, rot_dims // 2):
                raise KernelError("qk_norm_rope_store: cos and sin must be [tokens, rot_dims / 2] with rot_dims even and at most head_dim")
        for name, t in (("q_weight", q_weight), ("k_weight", k_weight)):
            if t is not None:
                self._need(t, name, torch.float32, 1)
                if t.shape[0] != head_dim:
                    raise KernelError(f"qk_norm_rope_store: {name} needs one entry per element of a head")
        if write_kv:
            self._need(slot_mapping, "slot_mapping", torch.int32, 1)
            for name, pool, d in (("k_pool", k_pool, head_dim), ("v_pool", v_pool, v_head_dim)):
                self._need(pool, name, z.dtype, 4)
                if tuple(pool.shape[1:]) != (num_kv_heads, page_size, d):
                    raise KernelError(f"qk_norm_rope_store: {name} is {list(pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {d}]")
        q = torch.empty((N, num_heads * head_dim), dtype=z.dtype, device=z.device)
        self._check(self.lib.llmie_qk_norm_rope_store(_ptr(z), z.shape[1], _ptr(q), _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps), _ptr(cos if rot_dims else None),
                                                      _ptr(sin if rot_dims else None), int(rot_dims), int(bool(interleaved)), _ptr(slot_mapping if write_kv else None),
                                                      _ptr(k_pool if write_kv else None), _ptr(v_pool if write_kv else None), N, num_heads, num_kv_heads, head_dim,
                                                      v_head_dim, page_size, int(bool(write_kv)), self._dt(z, "z"), self._stream()), "qk_norm_rope_store")
        return q

    # ------------------------------------------------------------------ mixers with a state of fixed size
    def causal_conv(self, z, col, channels, weight, bias, state, batch, activation=None):
        """A short causal convolution per channel over the rows of each request: ``y_t = act(bias + sum_j weight[:, j] u_(t - taps + 1 + j))``
        for the columns ``col .. col + channels`` of ``z``; inputs from before the step come out of ``state [slots, taps - 1, channels]``
        (float32), which is then moved on by the step's rows. ``batch`` is the step's context. Returns ``[N, channels]`` in z's type."""
        self._need(z, "z", None, 2)
        self._need(weight, "weight", torch.float32, 2)
        self._need(state, "state", torch.float32, 3)
        N = z.shape[0]
        taps = weight.shape[1]
        if weight.shape[0] != channels or col + channels > z.shape[1] or not 1 <= taps <= 8:
            raise KernelError("causal_conv: the weight does not fit the columns (or has more than 8 taps)")
        if tuple(state.shape[1:]) != (taps - 1, channels):
            raise KernelError(f"causal_conv: state is {list(state.shape)}, expected [slots, {taps - 1}, {channels}]")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
        if activation not in (None, "silu"):
            raise KernelError(f"causal_conv: activation '{activation}' is not built")
        out = torch.empty((N, channels), dtype=z.dtype, device=z.device)
        self._check(self.lib.llmie_causal_conv(ctypes.c_void_p(z.data_ptr() + col * z.element_size()), z.shape[1], channels, _ptr(weight), _ptr(bias),
                                               _ptr(state), _ptr(batch.seq_starts_dev), _ptr(batch.seq_slots), _ptr(out), channels, taps,
                                               1 if activation == "silu" else 0, batch.num_seqs, batch.max_seq_len, self._dt(z, "z"), self._stream()),
                    "causal_conv")
        return out

    def delta_rule(self, qkv, num_heads, num_kv_heads, head_dim, v_head_dim, a, b, b_col, A_log, dt_bias, state, batch, unit_eps=1e-6,
                   decay_per_head=False):
        """The gated delta rule with a decay per key channel over the rows of each request, from ``state [slots, heads, v_head_dim, head_dim]``
        (a head's ``S [head_dim, v_head_dim]`` kept column by column):
        ``qkv = [q: kv_heads x head_dim | k: the same | v: heads x v_head_dim]`` (after convolution and activation), ``a [N, heads * head_dim]``
        the decay's logits, ``b`` (columns from ``b_col``) the logits of beta. ``decay_per_head``: one decay per head, ``a [N, heads]``
        and ``dt_bias [heads]``. Returns float32 ``[N, heads * v_head_dim]``."""
        self._need(qkv, "qkv", None, 2)
        self._need(state, "state", torch.float32, 4)
        N = qkv.shape[0]
        H, G, D, DV = num_heads, num_kv_heads, head_dim, v_head_dim
        DA = 1 if decay_per_head else D
        if a.dim() != 2 or a.stride(1) != 1 or a.dtype != qkv.dtype or a.shape != (N, H * DA) or not a.is_cuda:
            raise KernelError("delta_rule: the decay's logits must be [rows, heads * head_dim] (or [rows, heads]) of the same type (they may be columns of wider rows)")
        if dt_bias.shape[0] != H * DA:
            raise KernelError("delta_rule: dt_bias needs one entry per decay")
        if qkv.shape[1] < 2 * G * D + H * DV or H % G or D > 256:
            raise KernelError("delta_rule: the rows do not fit the head sizes (head_dim at most 256)")
        if b.dim() != 2 or b.stride(1) != 1 or b.dtype != qkv.dtype or b_col + H > b.shape[1]:
            raise KernelError("delta_rule: the beta logits must be columns of rows of the same type")
        if tuple(state.shape[1:]) != (H, DV, D):
            raise KernelError(f"delta_rule: state is {list(state.shape)}, expected [slots, {H}, {DV}, {D}]")
        self._need(A_log, "A_log", torch.float32, 1)
        self._need(dt_bias, "dt_bias", torch.float32, 1)
        dev = qkv.device
        work = torch.empty((N, 2 * G * D + G + H * DA + H), dtype=torch.float32, device=dev)
        flat = work.view(-1)
        o = 0
        pieces = []
        for n in (N * G * D, N * G * D, N * H * DA, N * G, N * H):   # (rows of head_dim floats first: they start on 16-byte boundaries)
            pieces.append(flat[o:o + n])
            o += n
        qn, kn, decay, kq, beta = pieces
        dt = self._dt(qkv, "qkv")
        self._check(self.lib.llmie_delta_prepare(_ptr(qkv), qkv.shape[1], 0, G * D, _ptr(a), a.stride(0), ctypes.c_void_p(b.data_ptr() + b_col * b.element_size()),
                                                 b.stride(0), _ptr(A_log), _ptr(dt_bias), _ptr(qn), _ptr(kn), _ptr(kq), _ptr(decay), _ptr(beta), N, H, G, D,
                                                 ctypes.c_float(D ** -0.5), ctypes.c_float(unit_eps), int(bool(decay_per_head)), dt, self._stream()), "delta_rule (prepare)")
        out = torch.empty((N, H * DV), dtype=torch.float32, device=dev)
        self._check(self.lib.llmie_delta_scan(_ptr(qkv), qkv.shape[1], 2 * G * D, _ptr(qn), _ptr(kn), _ptr(kq), _ptr(decay), _ptr(beta), _ptr(state),
                                              _ptr(batch.seq_starts_dev), _ptr(batch.seq_slots), _ptr(out), H, G, D, DV, batch.num_seqs, batch.max_seq_len,
                                              int(bool(decay_per_head)), dt, self._stream()), "delta_rule (scan)")
        return out

    def ssm_scan(self, xbc, num_heads, groups, state_size, v_head_dim, dt, dt_col, A_log, dt_bias, skip, state, batch):
        """The state-space recurrence with one decay per head over the rows of each request, from ``state [slots, heads, v_head_dim,
        state_size]`` (a head's ``S [state_size, v_head_dim]`` kept column by column): ``xbc = [x: heads x v_head_dim | B: groups x state_size | C: the same]`` (after convolution and activation), ``dt``
        (columns from ``dt_col``) the step sizes' logits. Returns float32 ``[N, heads * v_head_dim]``."""
        self._need(xbc, "xbc", None, 2)
        self._need(state, "state", torch.float32, 4)
        H, G, NS, DV = num_heads, groups, state_size, v_head_dim
        if xbc.shape[1] != H * DV + 2 * G * NS or H % G or NS > 256:
            raise KernelError("ssm_scan: the rows do not fit the head sizes (state size at most 256)")
        if dt.dim() != 2 or dt.stride(1) != 1 or dt.dtype != xbc.dtype or dt_col + H > dt.shape[1]:
            raise KernelError("ssm_scan: the step sizes must be columns of rows of the same type")
        if tuple(state.shape[1:]) != (H, DV, NS):
            raise KernelError(f"ssm_scan: state is {list(state.shape)}, expected [slots, {H}, {DV}, {NS}]")
        for name, t in (("A_log", A_log), ("dt_bias", dt_bias), ("skip", skip)):
            self._need(t, name, torch.float32, 1)
            if t.shape[0] != H:
                raise KernelError(f"ssm_scan: {name} needs one entry per head")
        out = torch.empty((xbc.shape[0], H * DV), dtype=torch.float32, device=xbc.device)
        self._check(self.lib.llmie_ssm_scan(_ptr(xbc), xbc.shape[1], 0, H * DV, H * DV + G * NS, ctypes.c_void_p(dt.data_ptr() + dt_col * dt.element_size()),
                                            dt.stride(0), _ptr(A_log), _ptr(dt_bias), _ptr(skip), _ptr(state), _ptr(batch.seq_starts_dev), _ptr(batch.seq_slots),
                                            _ptr(out), H, G, NS, DV, batch.num_seqs, batch.max_seq_len, self._dt(xbc, "xbc"), self._stream()), "ssm_scan")
        return out

    def selective_scan(self, x, dt, bc, b_col, c_col, z, z_col, A_log, dt_bias, skip, state, batch):
        """The selective scan with a state per channel and state index over the rows of each request, from ``state [slots, channels,
        state_size]``: ``x [N, channels]`` (after convolution and activation), ``dt [N, channels]`` the step sizes' logits (``dt_bias`` is
        added and softplus taken here), ``bc`` rows that hold B from column ``b_col`` and C from ``c_col``, ``z`` (columns from ``z_col``)
        the gate; ``A_log [channels, state_size]``. Returns ``(y + skip x) silu(z)`` as ``[N, channels]`` in x's type."""
        self._need(x, "x", None, 2)
        self._need(dt, "dt", x.dtype, 2)
        self._need(state, "state", torch.float32, 3)
        self._need(A_log, "A_log", torch.float32, 2)
        N, C = x.shape
        NS = A_log.shape[1]
        if tuple(dt.shape) != (N, C) or A_log.shape[0] != C or NS > 256:
            raise KernelError("selective_scan: dt and A_log must match the channels (state size at most 256)")
        for name, t in (("dt_bias", dt_bias), ("skip", skip)):
            self._need(t, name, torch.float32, 1)
            if t.shape[0] != C:
                raise KernelError(f"selective_scan: {name} needs one entry per channel")
        for name, t, cols in (("bc", bc, max(b_col, c_col) + NS), ("z", z, z_col + C)):
            if t.dim() != 2 or t.stride(1) != 1 or t.dtype != x.dtype or t.shape[0] != N or cols > t.shape[1] or not t.is_cuda:
                raise KernelError(f"selective_scan: {name} must be rows of the same type that hold the columns asked for")
        if tuple(state.shape[1:]) != (C, NS):
            raise KernelError(f"selective_scan: state is {list(state.shape)}, expected [slots, {C}, {NS}]")
        out = torch.empty((N, C), dtype=x.dtype, device=x.device)
        self._check(self.lib.llmie_selective_scan(_ptr(x), x.stride(0), _ptr(dt), dt.stride(0), _ptr(bc), bc.stride(0), int(b_col), int(c_col),
                                                  ctypes.c_void_p(z.data_ptr() + z_col * z.element_size()), z.stride(0), _ptr(A_log), _ptr(dt_bias),
                                                  _ptr(skip), _ptr(state), _ptr(batch.seq_starts_dev), _ptr(batch.seq_slots), _ptr(out), C, NS,
                                                  batch.num_seqs, batch.max_seq_len, self._dt(x, "x"), self._stream()), "selective_scan")
        return out

    # ------------------------------------------------------------------ routed experts
    _SCORING = {"softmax": 0, "sigmoid": 1}

    def moe_route(self, logits, correction, top: int, scoring: str = "softmax"):
        """From float32 router logits ``[N, outputs]``: ``s = softmax(logits)``; the ``top`` outputs with the largest ``s + correction``
        (``correction`` may be None); returns ``(ids [N, top] int32, weights [N, top] float32)`` with the weights ``s / (sum of the chosen s + 1e-20)``.
        ``scoring="sigmoid"``: ``s = sigmoid(logits)`` and the weights are the chosen ``s`` as they are."""
        self._need(logits, "logits", torch.float32, 2)
        if scoring not in self._SCORING:
            raise KernelError(f"moe_route: scoring '{scoring}' is not built")
        N, total = logits.shape
        if correction is not None:
            self._need(correction, "correction", torch.float32, 1)
            if correction.shape[0] != total:
                raise KernelError("moe_route: the correction needs one entry per router output")
        if not 1 <= top <= total or total > 512:
            raise KernelError(f"moe_route: {top} of {total} router outputs cannot be chosen (at most 512 outputs)")
        ids = torch.empty((N, top), dtype=torch.int32, device=logits.device)
        weights = torch.empty((N, top), dtype=torch.float32, device=logits.device)
        self._check(self.lib.llmie_moe_route(_ptr(logits), _ptr(correction), _ptr(ids), _ptr(weights), N, total, top, self._SCORING[scoring], self._stream()), "moe_route")
        return ids, weights

    def moe_router(self, h, w_router, correction, top: int, scoring: str = "softmax"):
        """A router from the rows themselves: ``moe_route`` of the 32-bit logits ``h w_router^T`` (``h`` as it is stored). The few rows of
        a decode step, and float32 always, take one kernel that makes a token's logits and its choice (the sum over the inputs runs in one
        order whatever the step holds); prompt portions in bfloat16 take the tensor-core product with 32-bit output and the choice kernel."""
        self._need(h, "h", None, 2)
        self._need(w_router, "w_router", h.dtype, 2)
        if scoring not in self._SCORING:
            raise KernelError(f"moe_router: scoring '{scoring}' is not built")
        N, K = h.shape
        total = w_router.shape[0]
        fused = self.use_fused_router and (h.dtype == torch.float32 or N <= self.tc_max_rows) and (K + total + 4) * 4 <= 200 * 1024
        if not fused:
            return self.moe_route(self.linear(h, w_router, out_dtype=torch.float32), correction, top, scoring)
        if w_router.shape[1] != K:
            raise KernelError(f"moe_router: h has {K} columns, the router {w_router.shape[1]}")
        if correction is not None:
            self._need(correction, "correction", torch.float32, 1)
            if correction.shape[0] != total:
                raise KernelError("moe_router: the correction needs one entry per router output")
        if not 1 <= top <= total or total > 512:
            raise KernelError(f"moe_router: {top} of {total} router outputs cannot be chosen (at most 512 outputs)")
        ids = torch.empty((N, top), dtype=torch.int32, device=h.device)
        weights = torch.empty((N, top), dtype=torch.float32, device=h.device)
        self._check(self.lib.llmie_moe_router(_ptr(h), _ptr(w_router), _ptr(correction), _ptr(ids), _ptr(weights), N, K, total, top, self._SCORING[scoring],
                                              self._dt(h, "h"), self._stream()), "moe_router")
        return ids, weights

    def moe_experts(self, h, ids, weights, w_gate_up, w_down, add_to, glu=None, weight_inputs=False):
        """``add_to[t] += sum_k weights[t, k] * expert_(ids[t, k])(h[t])``: expert ``e < E`` is ``down_e(silu(gate_e x) * (up_e x))`` with
        ``w_gate_up [E, 2 F, K]`` (an expert's gate rows, then its up rows) and ``w_down [E, K, F]``; an id from ``E`` on is an identity
        expert whose output is ``h[t]`` itself. The (token, choice) pairs are sorted by expert on the device and every expert's rows go
        through its matrices as tiles of one grouped product. ``glu = (limit, alpha, shift)``: the experts are clamped units,
        ``down_e(g sigmoid(alpha g) (u + shift))`` with ``g = min(gate_e x, limit)``, ``u = clamp(up_e x, -limit, limit)``. ``weight_inputs``: the
        weight multiplies the expert's INPUT, ``add_to[t] += sum_k expert(weights[t, k] * h[t])`` (an identity expert then returns the weighted row)."""
        self.flush()
        limit, alpha, shift = (float(v) for v in glu) if glu is not None else (0.0, 1.0, 0.0)
        if glu is not None and not limit > 0:
            raise KernelError("moe_experts: the clamped unit needs a positive limit")
        fl = (ctypes.c_float(limit), ctypes.c_float(alpha), ctypes.c_float(shift))
        in_w = _ptr(weights if weight_inputs else None)
        self._need(h, "h", None, 2)
        self._need(add_to, "add_to", torch.float32, 2)
        self._need(ids, "ids", torch.int32, 2)
        self._need(weights, "weights", torch.float32, 2)
        self._need(w_gate_up, "w_gate_up", h.dtype, 3)
        self._need(w_down, "w_down", h.dtype, 3)
        N, K = h.shape
        top = ids.shape[1]
        E, F2, _ = w_gate_up.shape
        F = F2 // 2
        if tuple(w_gate_up.shape) != (E, 2 * F, K) or tuple(w_down.shape) != (E, K, F) or tuple(add_to.shape) != (N, K) or tuple(weights.shape) != (N, top) or ids.shape[0] != N:
            raise KernelError("moe_experts: the matrices, the choices and the rows do not fit each other")
        dev = h.device
        pairs = N * top
        dt = self._dt(h, "h")
        rows = min(self.lib.llmie_moe_tile_rows(K), self.lib.llmie_moe_tile_rows(F))
        # more than two rows per expert on average: the tensor cores, which fetch an expert's matrices once for up to 128 rows (the
        # CUDA-core product fetches them once per tile of at most 4; with one or two rows per expert both wait on the same bytes, and
        # the CUDA-core product spreads them over more blocks). The choice looks at sizes only, never at a count on the device
        tc = (self.use_tc_experts and h.dtype == torch.bfloat16 and K % 8 == 0 and F % 8 == 0 and pairs > 2 * E
              and w_gate_up.data_ptr() % 16 == 0 and w_down.data_ptr() % 16 == 0 and h.data_ptr() % 16 == 0)
        if not tc and rows < 1:
            raise KernelError(f"moe_experts: rows of {max(K, F)} numbers do not fit the shared memory of the product for few rows")
        tile_rows = self.lib.llmie_moe_grouped_tc_rows() if tc else rows
        max_tiles = -(-pairs // tile_rows) + E
        book = torch.empty((E + 1 + 2 * pairs + 1 + 2 * max_tiles,), dtype=torch.int32, device=dev)
        offsets, perm, place_of, tiles = book[:E + 1], book[E + 1:E + 1 + pairs], book[E + 1 + pairs:E + 1 + 2 * pairs], book[E + 1 + 2 * pairs:]
        self._check(self.lib.llmie_moe_sort(_ptr(ids), pairs, E, tile_rows, _ptr(offsets), _ptr(perm), _ptr(place_of), _ptr(tiles), max_tiles,
                                            self._stream()), "moe_experts (sort)")
        act = torch.empty((pairs, F), dtype=h.dtype, device=dev)
        y = torch.empty((pairs, K), dtype=torch.float32, device=dev)
        if tc:
            xs = torch.empty((pairs, K), dtype=h.dtype, device=dev)
            err = _ptr(self._errors(dev))
            self._check(self.lib.llmie_moe_gather(_ptr(h), _ptr(perm), _ptr(offsets), E, top, _ptr(xs), pairs, K, in_w, self._stream()), "moe_experts (gather)")
            self._check(self.lib.llmie_moe_grouped_tc(_ptr(xs), pairs, _ptr(w_gate_up), E, _ptr(offsets), _ptr(tiles), max_tiles, _ptr(act), F, K, 1,
                                                      self.num_sms, err, *fl, self._stream()), "moe_experts (gate and up, tcgen05)")
            self._check(self.lib.llmie_moe_grouped_tc(_ptr(act), pairs, _ptr(w_down), E, _ptr(offsets), _ptr(tiles), max_tiles, _ptr(y), K, F, 0,
                                                      self.num_sms, err, *fl, self._stream()), "moe_experts (down, tcgen05)")
        else:
            self._check(self.lib.llmie_moe_gemm(_ptr(h), _ptr(perm), top, _ptr(w_gate_up), _ptr(offsets), _ptr(tiles), max_tiles, _ptr(act), F, K, 1,
                                                tile_rows, in_w, *fl, dt, self._stream()), "moe_experts (gate and up)")
            self._check(self.lib.llmie_moe_gemm(_ptr(act), _ptr(None), 1, _ptr(w_down), _ptr(offsets), _ptr(tiles), max_tiles, _ptr(y), K, F, 0,
                                                tile_rows, _ptr(None), *fl, dt, self._stream()), "moe_experts (down)")
        # (with ``weight_inputs`` the sum is unweighted; the part refuses identity experts in that arrangement, whose rows would need the weight here)
        self._check(self.lib.llmie_moe_combine(_ptr(add_to), _ptr(y), _ptr(h), _ptr(place_of), _ptr(None if weight_inputs else weights), N, top, K, dt,
                                               self._stream()), "moe_experts (sum)")
        self._unfresh(add_to)

    # ------------------------------------------------------------------ latent attention
    def latent_prepare(self, z, q_rank, kv_rank, rot_dim, rot_dims, q_norm, kv_norm, eps, cos, sin, slot_mapping, kc_pool, page_size, write=True):
        """From ``z = [query latent | key/value latent | rotated part | ...]``: returns the normed query latent and, with
        ``write``, puts ``[normed key/value latent | turned rotated part]`` into the tokens' cache rows (one key/value head)."""
        self._need(z, "z", None, 2)
        N = z.shape[0]
        if z.shape[1] < q_rank + kv_rank + rot_dim:
            raise KernelError("latent_prepare: the rows are too short for the three parts")
        if q_rank:
            self._need(q_norm, "q_norm", torch.float32, 1)
        self._need(kv_norm, "kv_norm", torch.float32, 1)
        if (q_rank and q_norm.shape[0] != q_rank) or kv_norm.shape[0] != kv_rank:
            raise KernelError("latent_prepare: the norm weights do not match the ranks")
        if rot_dims:
            self._need(cos, "cos", torch.float32, 2)
            self._need(sin, "sin", torch.float32, 2)
            if tuple(cos.shape) != (N, rot_dims // 2) or tuple(sin.shape) != (N, rot_dims // 2):
                raise KernelError("latent_prepare: cos and sin must be [tokens, rot_dims / 2]")
        if write:
            self._need(slot_mapping, "slot_mapping", torch.int32, 1)
            self._need(kc_pool, "kc_pool", z.dtype, 4)
            if tuple(kc_pool.shape[1:]) != (1, page_size, kv_rank + rot_dim):
                raise KernelError(f"latent_prepare: the pool is {list(kc_pool.shape)}, expected [pages, 1, {page_size}, {kv_rank + rot_dim}]")
        cq = torch.empty((N, q_rank), dtype=z.dtype, device=z.device) if q_rank else None   # (q_rank 0: no query latent, the cache write alone)
        self._check(self.lib.llmie_latent_prepare(_ptr(z), z.shape[1], q_rank, kv_rank, rot_dim, rot_dims, _ptr(q_norm if q_rank else None), _ptr(kv_norm),
                                                  ctypes.c_float(eps), _ptr(cos), _ptr(sin), _ptr(slot_mapping), _ptr(kc_pool), page_size,
                                                  int(bool(write)), _ptr(cq), N, self._dt(z, "z"), self._stream()), "latent_prepare")
        return cq

    def latent_absorb(self, q, w_uk, cos, sin, num_heads, head_dim, rot_dim, rot_dims, kv_rank):
        """``q [N, heads * (head_dim + rot_dim)]`` -> ``[N, heads * (kv_rank + rot_dim)]``: every head's unrotated part times its
        ``[head_dim, kv_rank]`` block of ``w_uk`` (so that it meets the cached latents directly), its rotated part turned."""
        self._need(q, "q", None, 2)
        self._need(w_uk, "w_uk", q.dtype)
        N = q.shape[0]
        if q.shape[1] != num_heads * (head_dim + rot_dim) or w_uk.numel() != num_heads * head_dim * kv_rank:
            raise KernelError("latent_absorb: q or w_uk does not match the head sizes")
        out = torch.empty((N, num_heads * (kv_rank + rot_dim)), dtype=q.dtype, device=q.device)
        mode = 1
        if q.dtype == torch.bfloat16 and self.use_cublas and N >= self.head_matmul_library_rows:
            # many rows: the products of all heads as one batched library product (written straight into its columns of the
            # result); the kernel then only turns and copies the rotated parts
            torch.bmm(q.view(N, num_heads, head_dim + rot_dim)[:, :, :head_dim].transpose(0, 1), w_uk.view(num_heads, head_dim, kv_rank),
                      out=out.view(N, num_heads, kv_rank + rot_dim)[:, :, :kv_rank].transpose(0, 1))
            self.launches += 1
            mode = 3
        self._check(self.lib.llmie_head_matmul(_ptr(q), q.shape[1], head_dim + rot_dim, _ptr(w_uk), _ptr(out), out.shape[1], kv_rank + rot_dim,
                                               N, num_heads, head_dim, kv_rank, mode, rot_dim, rot_dims, _ptr(cos), _ptr(sin), _ptr(None), 0,
                                               self._dt(q, "q"), self._stream()), "latent_absorb")
        return out

    def latent_expand(self, o_lat, w_uv, gate, gate_col, num_heads, kv_rank, v_head_dim):
        """``o_lat [N, heads * kv_rank]`` -> ``[N, heads * v_head_dim]``: every head's row times its ``[kv_rank, v_head_dim]`` block of
        ``w_uv``, times ``sigmoid`` of the gate columns (from ``gate_col`` of ``gate``, one per output element; ``gate=None``: no gate)."""
        self._need(o_lat, "o_lat", None, 2)
        self._need(w_uv, "w_uv", o_lat.dtype)
        N = o_lat.shape[0]
        if o_lat.shape[1] != num_heads * kv_rank or w_uv.numel() != num_heads * kv_rank * v_head_dim:
            raise KernelError("latent_expand: o_lat or w_uv does not match the head sizes")
        if gate is not None:
            self._need(gate, "gate", o_lat.dtype, 2)
            if gate.shape[0] != N or gate_col + num_heads * v_head_dim > gate.shape[1]:
                raise KernelError("latent_expand: the gate columns lie outside the rows")
        out = torch.empty((N, num_heads * v_head_dim), dtype=o_lat.dtype, device=o_lat.device)
        mode = 2 if gate is not None else 0   # (no gate: the products alone; a gate per head was applied by the attention already)
        if o_lat.dtype == torch.bfloat16 and self.use_cublas and N >= self.head_matmul_library_rows:
            torch.bmm(o_lat.view(N, num_heads, kv_rank).transpose(0, 1), w_uv.view(num_heads, kv_rank, v_head_dim),
                      out=out.view(N, num_heads, v_head_dim).transpose(0, 1))
            self.launches += 1
            if gate is None:
                return out
            mode = 4   # the kernel only multiplies by the gate
        if gate is None:
            self._check(self.lib.llmie_head_matmul(_ptr(o_lat), o_lat.shape[1], kv_rank, _ptr(w_uv), _ptr(out), out.shape[1], v_head_dim, N,
                                                   num_heads, kv_rank, v_head_dim, mode, 0, 0, _ptr(None), _ptr(None), _ptr(None), 0,
                                                   self._dt(o_lat, "o_lat"), self._stream()), "latent_expand")
            return out
        self._check(self.lib.llmie_head_matmul(_ptr(o_lat), o_lat.shape[1], kv_rank, _ptr(w_uv), _ptr(out), out.shape[1], v_head_dim, N,
                                               num_heads, kv_rank, v_head_dim, mode, 0, 0, _ptr(None), _ptr(None),
                                               ctypes.c_void_p(gate.data_ptr() + gate_col * gate.element_size()), gate.shape[1],
                                               self._dt(o_lat, "o_lat"), self._stream()), "latent_expand")
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
