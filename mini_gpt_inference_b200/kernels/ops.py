"""The CUDA kernel set: what the parts call.

Each method checks its tensors (device, dtype, contiguity, shapes), allocates the output
with torch and launches a hand-written kernel of the library on torch's current stream.
torch is the tensor container and allocator here, nothing more: no torch operator
computes anything on this path.
"""

from __future__ import annotations

import ctypes
import weakref

import torch

from . import library
from .attention_plan import KEY_CHUNK, query_tiles
from .library import KernelLibraryError, check

EPILOGUES = {"none": 0, "gelu_tanh": 1, "residual": 2, "relu_sq": 3}
GATED_ACTIVATIONS = {"silu": 0, "clamped_swish": 1, "gelu_tanh": 2}     # the gated product of a unit's two halves
SKINNY_ROWS = 16         # most tokens the small-batch projection kernel takes
CLUSTER_ROWS = 128       # most tokens the mid-batch (K split over a cluster) projection kernel takes
CLUSTER_WIDE_MAX_BYTES = 3 << 20   # ... and the largest matrix it is given for more than 64 tokens
PREFETCH_MAX_BYTES = 32 << 20   # most of a following matrix that a streaming projection asks into L2
STREAM_MIN_ROWS = 8192   # a matrix this tall (the head) goes through the streaming kernel ...
STREAM_ROWS = 16         # ... for up to this many tokens (it takes 64; beyond 16 the tensor-core GEMM measured faster)


class DeferredNorm:
    """A LayerNorm that has not run yet: the projection that consumes it may fuse it into its
    prologue (small batches) or ask for it to be materialised.  ``rows`` optionally selects
    rows of ``x32`` first."""

    def __init__(self, ops, x32, gain, shift, eps, out_dtype, rows=None) -> None:
        self.ops, self.x32, self.gain, self.shift, self.eps = ops, x32, gain, shift, float(eps)
        self.dtype, self.rows = out_dtype, rows
        self.shape = (x32.shape[0] if rows is None else rows.numel(), x32.shape[1])
        self._rows_out = None      # the normalised rows, once a consumer asked for them (two consumers share them)

    def materialize(self):
        if self._rows_out is None:
            self._rows_out = self._materialize()
        return self._rows_out

    def _materialize(self):
        x = self.x32 if self.rows is None else self.ops.gather_rows(self.x32, self.rows)
        return self.ops.layernorm(x, self.gain, self.shift, self.eps, self.dtype)


class DeferredRMSNorm(DeferredNorm):
    """An RMS norm that has not run yet.  The projection kernels' prologues take it as a LayerNorm without a
    shift whose eps is negative (they then take no mean off), with ``offset + weight`` as the gain."""

    def __init__(self, ops, x32, weight, gain, eps, offset, out_dtype, rows=None) -> None:
        super().__init__(ops, x32, gain, None, -abs(float(eps)), out_dtype, rows)
        self.weight, self.offset = weight, float(offset)

    def _materialize(self):
        x = self.x32 if self.rows is None else self.ops.gather_rows(self.x32, self.rows)
        return self.ops.rmsnorm(x, self.weight, -self.eps, self.offset, self.dtype)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _ptr(t):
    return None if t is None else t.data_ptr()


class CudaOps:
    name = "cuda-sm100a"

    def __init__(self, device="cuda:0") -> None:
        if not torch.cuda.is_available():
            raise KernelLibraryError(
                "no CUDA device: this engine runs only on its sm_100a kernels and has no "
                "CPU path")
        self.device = torch.device(device)
        self.index = self.device.index or 0
        self.lib = library.load()
        torch.cuda.init()
        with torch.cuda.device(self.index):
            torch.empty(1, device=self.device)      # make sure the primary context exists
        arch = self.lib.mg_device_arch(self.index)
        if arch < 0:
            check(arch, "device query")
        if arch // 10 != 10:
            raise KernelLibraryError(
                f"device {self.index} has compute capability {arch / 10:.1f}; the kernels "
                "are built for sm_100a (NVIDIA B200) only")
        check(self.lib.mg_set_device(self.index), "set device")
        self.launches = 0          # kernels launched through this object
        # a guarded build (MINIGPT_B200_GUARDS=1): the kernels check the indices they read from device memory
        self.guards = bool(self.lib.mg_guards_enabled())
        # Kernels with bounded waits record a non-zero code here if a wait ran out.
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.use_tensor_cores = True
        self.use_split_attention = True
        self.use_skinny = True
        self.use_cluster = True
        self.use_stream = True
        self.use_wide = True
        # The large-matrix kernels also take any matrix of at least `stream_min_bytes` (None: only tall
        # ones, the head).  Measured with 8 tokens: a 5.1 MB matrix (1600 x 1600) is faster through
        # the kernel of tiled copies than through the small-batch kernel, matrices of 4.7 MB (3072 x
        # 768 and its transpose) are slower by a tenth; the boundary sits between them.  Where that
        # kernel refuses, the row-streaming kernel takes over, with rows cut into up to
        # `stream_max_chunks` K chunks (at 6400 columns, 67 chunks of 192 bytes, it was measured far
        # slower than the small-batch kernel, hence the limit).
        self.stream_min_bytes = 5_000_000
        self.stream_max_chunks = 8
        self.greedy_taken = False
        self.use_dependent_launch = True
        self.use_prefill_tc = True
        self.use_mma_attention = True
        self.use_chunked_memory = True     # prompt portions of the matrix-memory mixers chunk by chunk (bfloat16)
        self.use_recurrence_ranges = True  # long prompt portions of the gated recurrence with the warps sharing the tokens
        self.merge_ranges_in_last_cta = False
        self._counter_buf = None
        self._retired_counters = []
        self._sm_count = None
        self.use_fused_mlp = True
        # A streaming projection asks the weights of the projection that followed it the last time into
        # L2 once its own are on their way (learned from the order of the calls: a step repeats it).
        self.use_weight_prefetch = True
        self._last_weight = None   # data pointer of the matrix of the last projection
        self._next_weight = {}     # data pointer of a matrix -> weak reference to the matrix that came next
        self._packed = {}          # data pointer of a matrix -> (the matrix, its copy packed for a kernel)
        self._tile_lists = {}      # (rows, contexts, slots) of a step -> the prompt attention's work list
        self._ring = None          # (tensor that holds the residual stream, zeroed buffer, spare buffer)

    def begin_forward(self) -> None:
        """A forward pass begins: the first projection of a pass follows no other (the hint for the
        L2 prefetch never points from one pass, or one model, into another)."""
        self._last_weight = None

    # ---- helpers --------------------------------------------------------------------------
    def _run(self, code: int, what: str) -> None:
        """Check a launch's return code and count it."""
        check(code, what)
        self.launches += 1

    def _stream(self):
        # the raw handle of torch's current stream; the private getter costs a tenth of a
        # microsecond, building a Stream object two: it matters at sixty launches a step
        if _raw_stream is not None:
            return _raw_stream(self.index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _want(self, t, dtype, name, dims=None):
        if t.device != self.device:
            raise KernelLibraryError(f"{name}: tensor on {t.device}, kernels run on {self.device}")
        if dtype is not None and t.dtype != dtype:
            raise KernelLibraryError(f"{name}: dtype {t.dtype}, expected {dtype}")
        if not t.is_contiguous():
            raise KernelLibraryError(f"{name}: tensor must be contiguous")
        if dims is not None and t.dim() != dims:
            raise KernelLibraryError(f"{name}: expected {dims} dims, got shape {tuple(t.shape)}")
        return t

    @staticmethod
    def _is_bf16(t) -> int:
        if t.dtype == torch.bfloat16:
            return 1
        if t.dtype == torch.float32:
            return 0
        raise KernelLibraryError(f"dtype {t.dtype} is neither bfloat16 nor float32")

    def _counters(self, count: int):
        """Zeroed ints that the split attention kernel uses to find its last block per row and
        leaves zeroed; kept for the life of the object, grown on demand (a buffer that was
        handed out once is never freed)."""
        if self._counter_buf is None or self._counter_buf.numel() < count:
            if self._counter_buf is not None:
                # A captured graph may hold the old buffer's address: it stays alive (and zeroed,
                # as its kernels leave it) for as long as this object does.
                self._retired_counters.append(self._counter_buf)
            self._counter_buf = torch.zeros(max(count, 4096, 2 * (self._counter_buf.numel()
                                                                   if self._counter_buf is not None else 0)),
                                            dtype=torch.int32, device=self.device)
        return self._counter_buf

    def set_dependent_launch(self, on: bool) -> None:
        """Let kernels that support it start while the kernel before them drains (used while a
        decode step is captured into a CUDA graph)."""
        check(self.lib.mg_set_dependent_launch(1 if (on and self.use_dependent_launch) else 0),
              "set_dependent_launch")

    def check_indices(self) -> None:
        """Guarded builds: raise if a kernel met a token id, position, cache row, page, request or row
        number outside its table since the last call (synchronises; the kernel skipped the access
        or read index 0 in its place, so the results of that step are invalid but no memory
        outside a table was touched).  Ordinary builds: nothing to ask."""
        if not self.guards:
            return
        torch.cuda.synchronize(self.device)
        record = (ctypes.c_longlong * 4)()
        faults = []
        for name in library.GUARDED_FILES:
            check(getattr(self.lib, f"mg_{name}_index_fault")(record), "index guard")
            if record[0]:
                what = library.GUARD_CODES.get(int(record[0]), f"index (code {record[0]})")
                faults.append(f"{name}: {what} {record[2]} is outside 0..{record[3] - 1} (block {record[1]})")
        if faults:
            raise KernelLibraryError("a kernel met an index outside its table: " + "; ".join(faults))

    def check_status(self) -> None:
        """Raise if a kernel reported that one of its bounded waits ran out (synchronises); in a
        guarded build also if one met an index outside its table."""
        self.check_indices()
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise KernelLibraryError(f"a kernel gave up waiting (code {code}); its results are invalid")

    def wait_probe(self, limit: int = 1000) -> None:
        """Run a kernel whose bounded wait runs out (it waits ``limit`` tries on a barrier that is
        never completed, with the wait all kernels share) and records its code in the status
        word: what ``check_status`` and the engine then do can be seen without any fault."""
        self._run(self.lib.mg_wait_probe(int(limit), _ptr(self.status), self._stream()), "wait probe")

    def status_to_host(self, pinned=None):
        """Queue a copy of the status word into pinned host memory on the current stream and
        return that memory; once the stream has been synchronised (or an event recorded after
        this call has), ``raise_on_status(pinned)`` tells whether a kernel before it gave up."""
        if pinned is None:
            pinned = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        pinned.copy_(self.status, non_blocking=True)
        return pinned

    def raise_on_status(self, pinned) -> None:
        self.check_indices()
        code = int(pinned[0])
        if code != 0:
            self.status.zero_()
            raise KernelLibraryError(f"a kernel gave up waiting (code {code}); its results are invalid")

    # ---- embedding and norms --------------------------------------------------------------------
    def embed(self, token_ids, positions, tok_emb, pos_table, source=None, previous=None, scale=1.0):
        """Rows of the embedding times ``scale`` (plus rows of the position table).  With ``source``:
        a row whose source is >= 0 takes its id from ``previous[source]`` instead of ``token_ids``."""
        self._want(token_ids, torch.int32, "token_ids", 1)
        self._want(positions, torch.int32, "positions", 1)
        if source is not None:
            self._want(source, torch.int32, "token sources", 1)
            self._want(previous, torch.int32, "previous ids", 1)
            if source.numel() != token_ids.numel():
                raise KernelLibraryError("embed: one source per token")
        self._want(tok_emb, None, "tok_emb", 2)
        if pos_table is not None:
            self._want(pos_table, tok_emb.dtype, "pos_table", 2)
            if pos_table.shape[1] != tok_emb.shape[1]:
                raise KernelLibraryError("embed: position table and embedding differ in width")
        n, width = token_ids.numel(), tok_emb.shape[1]
        out = torch.empty((n, width), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_embed(_ptr(token_ids), _ptr(positions), _ptr(tok_emb), _ptr(pos_table),
                                _ptr(out), n, width, self._is_bf16(tok_emb), _ptr(source), _ptr(previous),
                                tok_emb.shape[0], pos_table.shape[0] if pos_table is not None else 0,
                                previous.numel() if previous is not None else 0, float(scale), self._stream()),
              "embed")
        return out

    def layernorm(self, x32, gain, shift, eps, out_dtype):
        self._want(x32, torch.float32, "layernorm input", 2)
        self._want(gain, torch.float32, "layernorm gain", 1)
        if shift is not None:
            self._want(shift, torch.float32, "layernorm shift", 1)
        rows, width = x32.shape
        if gain.numel() != width:
            raise KernelLibraryError("layernorm: gain does not match the width")
        out = torch.empty((rows, width), dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_layernorm(_ptr(x32), _ptr(gain), _ptr(shift), _ptr(out), rows, width,
                                    float(eps), self._is_bf16(out), self._stream()), "layernorm")
        return out

    def rmsnorm(self, x32, weight, eps, offset, out_dtype):
        """``x / sqrt(mean(x^2) + eps) * (offset + weight)``, statistics in 32-bit."""
        self._want(x32, torch.float32, "rmsnorm input", 2)
        self._want(weight, torch.float32, "rmsnorm weight", 1)
        rows, width = x32.shape
        if weight.numel() != width:
            raise KernelLibraryError("rmsnorm: the weight does not match the width")
        out = torch.empty((rows, width), dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_rmsnorm(_ptr(x32), _ptr(weight), _ptr(out), rows, width, float(eps), float(offset),
                                      self._is_bf16(out), self._stream()), "rmsnorm")
        return out

    def defer_rmsnorm(self, x32, weight, eps, offset, out_dtype, rows=None):
        """An RMS norm to be fused into the projection that consumes it, where that pays."""
        self._want(x32, torch.float32, "rmsnorm input", 2)
        gain = weight
        if offset != 0.0:
            hit = self._packed.get(("rms gain", weight.data_ptr(), float(offset)))
            if hit is None or hit[0] is not weight:
                hit = (weight, (weight + float(offset)).contiguous())     # made once, when a weight is first seen
                self._packed[("rms gain", weight.data_ptr(), float(offset))] = hit
            gain = hit[1]
        return DeferredRMSNorm(self, x32, weight, gain, eps, offset, out_dtype, rows)

    def clone(self, x):
        """A copy of a tensor (a device-to-device copy on the current stream)."""
        return x.clone()

    def concat_cast(self, a32, b32, out_dtype):
        """``[a ; b]`` row by row, two 32-bit tensors of one shape, in ``out_dtype``."""
        self._want(a32, torch.float32, "first rows", 2)
        self._want(b32, torch.float32, "second rows", 2)
        if a32.shape != b32.shape:
            raise KernelLibraryError("concat: the two tensors differ in shape")
        rows, width = a32.shape
        out = torch.empty((rows, 2 * width), dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_concat_cast(_ptr(a32), _ptr(b32), _ptr(out), rows, width, self._is_bf16(out),
                                          self._stream()), "concat")
        return out

    def embed_pairs(self, ctx, tok_emb, pair_emb, pos_table, buckets, mul_prev, mul_cur, state, source=None,
                    previous=None):
        """Rows of the embedding plus rows of the token-pair table (row ``(previous id * mul_prev + id *
        mul_cur) mod buckets``, row ``buckets`` for a request's first token) plus rows of the position table.
        ``state``: int32 ``[slots, 1]``, the last token each request brought (read for a step's first token of
        a request that has tokens in the cache, written for every request of the step)."""
        self._want(ctx.token_ids, torch.int32, "token_ids", 1)
        self._want(ctx.positions, torch.int32, "positions", 1)
        self._want(tok_emb, None, "tok_emb", 2)
        self._want(pair_emb, tok_emb.dtype, "pair table", 2)
        self._want(state, torch.int32, "last tokens", 2)
        if pos_table is not None:
            self._want(pos_table, tok_emb.dtype, "pos_table", 2)
        if source is not None:
            self._want(source, torch.int32, "token sources", 1)
            self._want(previous, torch.int32, "previous ids", 1)
        n, width = ctx.token_ids.numel(), tok_emb.shape[1]
        if pair_emb.shape != (buckets + 1, width) or (pos_table is not None and pos_table.shape[1] != width):
            raise KernelLibraryError("embed_pairs: the tables do not fit")
        if not (0 <= int(mul_prev) < 2 ** 31 and 0 <= int(mul_cur) < 2 ** 31 and 0 < int(buckets) < 2 ** 31):
            raise KernelLibraryError("embed_pairs: buckets and multipliers must fit 31 bits")
        out = torch.empty((n, width), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_embed_pairs(
            _ptr(ctx.token_ids), _ptr(ctx.positions), _ptr(ctx.token_request), _ptr(ctx.req_q_start), _ptr(ctx.req_q_len),
            _ptr(ctx.req_ctx_before), _ptr(ctx.req_state_slot), _ptr(tok_emb), _ptr(pair_emb), _ptr(pos_table), _ptr(out),
            _ptr(state), state.shape[1], n, width, self._is_bf16(tok_emb), _ptr(source), _ptr(previous), tok_emb.shape[0],
            pos_table.shape[0] if pos_table is not None else 0, previous.numel() if previous is not None else 0,
            int(buckets), int(mul_prev), int(mul_cur), ctx.req_q_start.numel(), state.shape[0], self._stream()),
            "embed_pairs")
        return out

    # ---- mixers with a matrix memory ------------------------------------------------------------------
    MEMORY_CHUNK_MIN_TOKENS = 32     # a step whose longest portion is shorter runs the token-by-token scan

    def _memory_chunks_name(self, head_dim, v_dim, mlstm):
        tokens = self.lib.mg_matrix_memory_chunk_tokens(int(head_dim), int(v_dim), 1 if mlstm else 0)
        return (f"memory_chunks/{tokens}", tokens) if tokens > 0 else (None, 0)

    def plan_memory_chunks(self, batch, plan, head_dim, v_dim, mlstm) -> None:
        """Host half of the chunked scan of the matrix-memory mixers: the step's tokens cut into chunks, request
        by request (``[chunks, 4]``: request, first row, tokens, 0) and each request's range of chunks
        (``[requests, 2]``), under a name that layers with the same chunk length share.  Nothing is planned
        for 32-bit steps (the token-by-token scan has one fixed order of sums whatever the cut) and for steps
        of short portions."""
        if (not self.use_chunked_memory or batch.act_dtype != torch.bfloat16
                or max(batch.q_len) < self.MEMORY_CHUNK_MIN_TOKENS):
            return
        name, tokens = self._memory_chunks_name(head_dim, v_dim, mlstm)
        if name is None or name in plan.arrays:
            return
        import numpy as np

        chunks, ranges, row = [], [], 0
        for r, n in enumerate(batch.q_len):
            ranges.append((len(chunks), -(-n // tokens)))
            for first in range(0, n, tokens):
                chunks.append((r, row + first, min(tokens, n - first), 0))
            row += n
        plan.arrays[name] = np.asarray(chunks, dtype=np.int32).reshape(-1, 4)
        plan.arrays[name + "/requests"] = np.asarray(ranges, dtype=np.int32).reshape(-1, 2)
        plan.signature.append(("memory_chunks", tokens))

    MEMORY_MODES = {"gla": 0, "mlstm": 1, "ssd": 2, "retention": 3, "wkv": 4}

    def matrix_memory_scan(self, ctx, mode, proj, q_off, k_off, v_off, n_head, head_dim, v_dim, gates, constant, state,
                           state_offset=0, qk_group=1, head_consts=None):
        """The scan of a mixer with a matrix memory over the step's tokens, request by request, from and to
        the requests' state slots.  ``mode`` ``"gla"``: ``gates`` are the decays' pre-activations
        ``[tokens, n_head * head_dim]`` and ``constant`` is tau; ``"mlstm"``: ``gates`` are the input and
        forget gates' pre-activations ``[tokens, 2 * n_head]`` and ``constant`` is their cap.  Returns
        ``(o [tokens, n_head * v_dim] 32-bit, aux)``; ``aux`` (mlstm) holds ``n . q`` and ``m`` per token
        and head for the division that ``head_norm_gate`` does.

        ``"ssd"`` (state-space duality, Mamba-2): ``S <- exp(-exp(A_h) dt) S + dt k v^T``, ``o = S^T q + D_h v`` with
        ``dt = softplus(gates[:, h])``, q and k unscaled and shared by ``qk_group`` neighbouring heads, and
        ``head_consts`` = ``[A_0 .. A_(H-1), D_0 .. D_(H-1)]`` (32-bit).  ``state_offset``: where in a slot the
        memories begin (a mixer may keep something else in front of them).

        ``"retention"``: ``S <- a_h S + (k / sqrt(head_dim)) v^T`` with the fixed decays ``head_consts`` ``[n_head]``, no
        gates (``None``), q unscaled.  ``"wkv"``: ``o = (S + diag(u) k v^T)^T q`` read before ``S <- diag(w) S + k v^T``,
        ``w = exp(-exp(gates))`` per key channel, ``head_consts`` the bonus ``u`` ``[n_head * head_dim]``.  ``proj`` may
        be ``[planes, tokens, columns]`` (q, k, v from projections of their own): an offset is then
        ``plane * tokens * columns + column``."""
        planes = proj.dim() == 3
        self._want(proj, None, "projection rows", 3 if planes else 2)
        if gates is not None or mode != "retention":
            self._want(gates, torch.float32, "gates", 2)
        self._want(state, torch.float32, "state slots", 2)
        if mode not in self.MEMORY_MODES:
            raise KernelLibraryError(f"matrix memory: mode {mode!r}")
        if mode in ("retention", "wkv"):
            want = n_head if mode == "retention" else n_head * head_dim
            if head_consts is None or self._want(head_consts, torch.float32, "per-head constants", 1).numel() != want:
                raise KernelLibraryError(f"matrix memory: the {mode} form wants {want} per-head constants")
        if mode == "ssd" and (head_consts is None or self._want(head_consts, torch.float32, "per-head constants", 1).numel() != 2 * n_head):
            raise KernelLibraryError("matrix memory: the state-space form wants A and D of every head")
        cols_needed = n_head * (v_dim + (1 if mode == "mlstm" else 0)) * head_dim + (n_head if mode == "mlstm" else 0)
        if state_offset < 0 or state_offset + cols_needed > state.shape[1]:
            raise KernelLibraryError("matrix memory: the state slots are too small")
        n, ld = proj.shape[-2], proj.shape[-1]
        if gates is not None and gates.shape[0] != n:
            raise KernelLibraryError("matrix memory: one row of gates per token")
        gates_ld = gates.shape[1] if gates is not None else 0
        form = self.MEMORY_MODES[mode] if mode in ("retention", "wkv") else 0
        mlstm = mode == "mlstm"
        out = torch.empty((n, n_head * v_dim), dtype=torch.float32, device=self.device)
        aux = torch.empty((n, n_head, 2), dtype=torch.float32, device=self.device) if mlstm else None
        name, tokens = self._memory_chunks_name(head_dim, v_dim, mlstm)
        chunks = getattr(ctx, "extra", {}).get(name) if name is not None else None
        if chunks is not None and chunks.shape[0] > 0 and self.use_chunked_memory:
            # a step with prompt portions: chunk by chunk (three kernels, every SM at work)
            ranges = ctx.extra[name + "/requests"]
            cols = v_dim + (1 if mlstm else 0)
            cum = torch.empty((n, n_head, 2 if mlstm else head_dim), dtype=torch.float32, device=self.device)
            chunk_state = torch.empty((chunks.shape[0], n_head, cols, head_dim), dtype=torch.float32, device=self.device)
            meta = torch.empty((chunks.shape[0], n_head, 4), dtype=torch.float32, device=self.device) if mlstm else None
            self._run(self.lib.mg_matrix_memory_chunked(
                _ptr(proj), ld, q_off, k_off, v_off, _ptr(gates), gates_ld, _ptr(chunks), _ptr(ranges),
                _ptr(ctx.req_ctx_before), _ptr(ctx.req_state_slot), state.data_ptr() + 4 * int(state_offset), state.shape[1],
                _ptr(cum), _ptr(chunk_state), _ptr(meta), _ptr(out), _ptr(aux), chunks.shape[0], tokens, ranges.shape[0], n,
                n_head, head_dim, v_dim, float(constant), 1 if mlstm else 0, state.shape[0], self._is_bf16(proj),
                int(qk_group), _ptr(head_consts) if mode in ("ssd", "retention", "wkv") else None, form, self._stream()),
                "matrix memory (chunks)")
            self.launches += 2
            return out, aux
        self._run(self.lib.mg_matrix_memory_scan(
            _ptr(proj), ld, q_off, k_off, v_off, _ptr(gates), gates_ld, _ptr(ctx.req_q_start),
            _ptr(ctx.req_q_len), _ptr(ctx.req_ctx_before), _ptr(ctx.req_state_slot), state.data_ptr() + 4 * int(state_offset),
            state.shape[1], _ptr(out), _ptr(aux), ctx.req_q_start.numel(), n, n_head, head_dim, v_dim, float(constant),
            self.MEMORY_MODES[mode], state.shape[0], self._is_bf16(proj), int(qk_group), _ptr(head_consts), self._stream()),
            "matrix memory scan")
        return out, aux

    def head_norm_gate(self, out32, aux, gate, gain, n_head, v_dim, eps, per_head_gain, gate_activation, out_dtype,
                       positions=None):
        """Every head of ``out32`` (divided by ``max(|n . q|, exp(-m)) + 1e-6`` from ``aux`` if given) divided by
        its root mean square, times ``gain`` (``[v_dim]``, or ``[n_head * v_dim]`` if ``per_head_gain``), times
        ``silu`` or ``sigmoid`` of ``gate`` (a 2-D view of ``n_head * v_dim`` columns), in ``out_dtype``.  Rows whose
        ``positions`` entry is negative (padding) become zeros."""
        self._want(out32, torch.float32, "memory output", 2)
        if gain is not None:
            self._want(gain, torch.float32, "head gain", 1)
        n = out32.shape[0]
        if (gate.dtype != out_dtype or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape != (n, n_head * v_dim)
                or out32.shape[1] != n_head * v_dim
                or (gain is not None and gain.numel() != (n_head * v_dim if per_head_gain else v_dim))):
            raise KernelLibraryError("head_norm_gate: shapes do not fit")
        if gate_activation not in ("silu", "sigmoid"):
            raise KernelLibraryError(f"head_norm_gate: gate activation {gate_activation!r}")
        if positions is not None and self._want(positions, torch.int32, "positions", 1).numel() != n:
            raise KernelLibraryError("head_norm_gate: one position per row")
        out = torch.empty((n, n_head * v_dim), dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_head_norm_gate(_ptr(out32), _ptr(aux), _ptr(gate), gate.stride(0), _ptr(gain), _ptr(positions),
                                             _ptr(out), n, n_head, v_dim, float(eps), 1 if per_head_gain else 0,
                                             1 if gate_activation == "sigmoid" else 0, self._is_bf16(out), self._stream()),
                  "head_norm_gate")
        return out

    def gather_rows(self, x32, rows):
        self._want(x32, torch.float32, "gather input", 2)
        self._want(rows, torch.int32, "rows", 1)
        out = torch.empty((rows.numel(), x32.shape[1]), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_gather_rows(_ptr(x32), _ptr(rows), _ptr(out), rows.numel(), x32.shape[1],
                                      x32.shape[0], self._stream()), "gather_rows")
        return out

    def gather_tokens(self, token_ids, source, previous):
        """token_ids[i] = previous[source[i]] for rows with source[i] >= 0 (in place): the tokens a
        step sampled become the next step's inputs without passing through the host."""
        for name, t in (("token_ids", token_ids), ("source", source), ("previous", previous)):
            self._want(t, torch.int32, name, 1)
        self._run(self.lib.mg_gather_tokens(_ptr(token_ids), _ptr(source), _ptr(previous),
                                            token_ids.numel(), previous.numel(), self._stream()), "gather_tokens")

    def upload_ints(self, dst, pinned) -> None:
        """dst[:] = pinned[:] where ``pinned`` is page-locked host memory: the device reads it
        itself, so nothing switches engines between this and the kernels that follow."""
        self._want(dst, torch.int32, "upload destination", 1)
        if (pinned.dtype != torch.int32 or pinned.device.type != "cpu" or not pinned.is_pinned()
                or pinned.numel() != dst.numel() or not pinned.is_contiguous()):
            raise KernelLibraryError("upload_ints: the source must be pinned int32 host memory of the same size")
        self._run(self.lib.mg_copy_ints(_ptr(dst), _ptr(pinned), dst.numel(), self._stream()), "upload_ints")

    # ---- projections ----------------------------------------------------------------------------
    def defer_layernorm(self, x32, gain, shift, eps, out_dtype, rows=None):
        """A LayerNorm to be fused into the projection that consumes it, where that pays."""
        self._want(x32, torch.float32, "layernorm input", 2)
        return DeferredNorm(self, x32, gain, shift, eps, out_dtype, rows)

    def _skinny_ok(self, m, k, dtype) -> bool:
        return (self.use_skinny and dtype == torch.bfloat16 and 0 < m <= SKINNY_ROWS and k % 8 == 0
                and SKINNY_ROWS * (2 * k + 64) + 8 * SKINNY_ROWS * 8 * 4 + 8 * k <= 200 * 1024)

    @staticmethod
    def _sink_args(kv_sink):
        """The key/value sink of a QKV projection as the C functions take it."""
        if kv_sink is None:
            return [None, None, None, 0, 0, 0, 0, 0]
        cache, slots, n_head, n_kv_head, head_dim = kv_sink
        return [_ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(slots), n_head * head_dim, n_kv_head,
                head_dim, cache.page_tokens, cache.k_pages.shape[0]]

    def _linear(self, x, weight, bias, epilogue, out, residual, kv_sink=None, greedy=None):
        """x: a tensor [M, K] or a DeferredNorm.  kv_sink: (cache view, slots, n_head, n_kv_head,
        head_dim) to also write key/value features to the cache.  greedy: (ids out, vocabulary
        limit) to also leave each row's argmax where the kernel that runs can take it on its way
        (``self.greedy_taken`` says whether it did).  Returns True if the sink was served inside
        the projection kernel."""
        deferred = x if isinstance(x, DeferredNorm) else None
        m, k = x.shape
        n = weight.shape[0]
        self._want(weight, None, "linear weight", 2)
        # which matrix followed which the last time: what a streaming kernel asks into L2 on its way
        if self._last_weight is not None:
            self._next_weight[self._last_weight] = weakref.ref(weight)
        self._last_weight = weight.data_ptr()
        if bias is not None:
            self._want(bias, torch.float32, "linear bias", 1)
        if weight.shape[1] != k or (bias is not None and bias.numel() != n):
            raise KernelLibraryError(
                f"linear: shapes do not fit: x {tuple(x.shape)}, w {tuple(weight.shape)}")
        out_bf16 = self._is_bf16(out) if out is not None else 0
        large = n >= STREAM_MIN_ROWS or (self.stream_min_bytes is not None and 2 * n * k >= self.stream_min_bytes)
        if self.use_wide and weight.dtype == torch.bfloat16 and 0 < m <= SKINNY_ROWS and k % 8 == 0 and large:
            # a matrix of many megabytes: whole rows as TMA boxes through a ring of stages, the first of
            # them asked for before the dependency wait
            if deferred is not None:
                args = [None, _ptr(deferred.x32), _ptr(deferred.rows), _ptr(deferred.gain),
                        _ptr(deferred.shift), deferred.eps]
            else:
                self._want(x, weight.dtype, "linear input", 2)
                args = [_ptr(x), None, None, None, None, 0.0]
            amax, parts = [None, None, 0], 0
            if greedy is not None:
                ids_out, limit = greedy
                parts = self.lib.mg_linear_wide_parts(m, n, k, 1 if deferred is not None else 0)
                part_v = torch.empty((m * parts,), dtype=torch.float32, device=self.device)
                part_i = torch.empty((m * parts,), dtype=torch.int32, device=self.device)
                amax = [_ptr(part_v), _ptr(part_i), int(limit or 0)]
            follower = self._next_weight.get(weight.data_ptr())
            follower = follower() if follower is not None and self.use_weight_prefetch else None
            ahead = [None, 0]
            if follower is not None and follower.is_cuda and follower.data_ptr() % 128 == 0:
                ahead = [_ptr(follower), min(follower.numel() * follower.element_size(), PREFETCH_MAX_BYTES) // 128]
            code = self.lib.mg_linear_wide(*args, _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                           m, n, k, epilogue, out_bf16, *self._sink_args(kv_sink), *amax,
                                           *ahead, _ptr(self.status), self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (large matrix)")
                if greedy is not None:
                    self._run(self.lib.mg_argmax_merge(_ptr(part_v), _ptr(part_i), _ptr(ids_out), m, parts,
                                                       self._stream()), "argmax (merge)")
                    self.greedy_taken = True
                return kv_sink is not None
        if (self.use_stream and weight.dtype == torch.bfloat16 and 0 < m <= STREAM_ROWS and k % 8 == 0 and large):
            # a tall matrix (the head) or one of many megabytes: one CTA per SM streams it through
            # shared memory
            if deferred is not None and m > SKINNY_ROWS:
                # more rows than a CTA normalises quickly: the norm runs as a kernel of its own
                x, deferred = deferred.materialize(), None
            if deferred is not None:
                args = [None, _ptr(deferred.x32), _ptr(deferred.rows), _ptr(deferred.gain),
                        _ptr(deferred.shift), deferred.eps]
            else:
                self._want(x, weight.dtype, "linear input", 2)
                args = [_ptr(x), None, None, None, None, 0.0]
            amax = [None, None, 0]
            if greedy is not None:
                ids_out, limit = greedy
                parts = self.lib.mg_linear_stream_parts(n)
                part_v = torch.empty((m * parts,), dtype=torch.float32, device=self.device)
                part_i = torch.empty((m * parts,), dtype=torch.int32, device=self.device)
                amax = [_ptr(part_v), _ptr(part_i), int(limit or 0)]
            code = self.lib.mg_linear_stream(*args, _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                             m, n, k, epilogue, out_bf16, *self._sink_args(kv_sink), *amax,
                                             self.stream_max_chunks, _ptr(self.status), self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (wide matrix)")
                if greedy is not None:
                    self._run(self.lib.mg_argmax_merge(_ptr(part_v), _ptr(part_i), _ptr(ids_out), m, parts,
                                                       self._stream()), "argmax (merge)")
                    self.greedy_taken = True
                return kv_sink is not None
        if self._skinny_ok(m, k, weight.dtype):
            sink = self._sink_args(kv_sink)
            if deferred is not None:
                args = [None, _ptr(deferred.x32), _ptr(deferred.rows), _ptr(deferred.gain),
                        _ptr(deferred.shift), deferred.eps]
            else:
                self._want(x, weight.dtype, "linear input", 2)
                args = [_ptr(x), None, None, None, None, 0.0]
            amax = [None, None, 0]
            if greedy is not None:
                # first stage of the argmax over the rows, on the projection's way
                ids_out, limit = greedy
                parts = self.lib.mg_linear_skinny_ctas(n, k)
                part_v = torch.empty((m * parts,), dtype=torch.float32, device=self.device)
                part_i = torch.empty((m * parts,), dtype=torch.int32, device=self.device)
                amax = [_ptr(part_v), _ptr(part_i), int(limit or 0)]
            code = self.lib.mg_linear_skinny(*args, _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                             m, n, k, epilogue, out_bf16, *sink, *amax, self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (small batch)")
                if greedy is not None:
                    self._run(self.lib.mg_argmax_merge(_ptr(part_v), _ptr(part_i), _ptr(ids_out), m, parts,
                                                       self._stream()), "argmax (merge)")
                    self.greedy_taken = True
                return kv_sink is not None
        if deferred is not None:
            x = deferred.materialize()
        self._want(x, weight.dtype, "linear input", 2)
        # (a matrix of thousands of 8-row tiles, the head, is left to the tensor-core GEMM: every one
        # of its clusters would stage the activations and meet at a barrier for a few KB of weights)
        # (and beyond 64 tokens it keeps only matrices of up to 3 MB: measured with 96 and 128 tokens, it
        # is faster than the tensor-core GEMM at 512 x 2048, slower from 3 x 768 x 768 elements on)
        if (x.dtype == torch.bfloat16 and self.use_cluster and 0 < m <= CLUSTER_ROWS and k % 8 == 0
                and n <= 8192 and (m <= 64 or 2 * n * k <= CLUSTER_WIDE_MAX_BYTES)):
            sink = self._sink_args(kv_sink)
            code = self.lib.mg_linear_cluster(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                              m, n, k, epilogue, out_bf16, *sink, self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (mid batch)")
                return kv_sink is not None
        if x.dtype == torch.bfloat16 and self.use_tensor_cores:
            # the key/value copy moves 16 bytes at a time: head sizes that are multiples of 8
            fused = kv_sink is not None and kv_sink[4] % 8 == 0
            sink = self._sink_args(kv_sink if fused else None)
            code = self.lib.mg_linear_tc(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                         m, n, k, epilogue, out_bf16, *sink, _ptr(self.status),
                                         self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "linear (tensor cores)")
                return fused
        self._run(self.lib.mg_linear_simt(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _ptr(residual),
                                      m, n, k, epilogue, self._is_bf16(x), out_bf16, self._stream()),
              "linear")
        return False

    def linear(self, x, weight, bias, activation, out_dtype, out=None):
        """``act(x W^T + bias)`` in ``out_dtype``; ``out``: a contiguous tensor of that shape and type to write into."""
        if activation not in ("none", "gelu_tanh", "relu_sq"):
            raise KernelLibraryError(f"linear: no epilogue for activation {activation!r}")
        if out is None:
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=self.device)
        elif out.shape != (x.shape[0], weight.shape[0]) or self._want(out, out_dtype, "linear output", 2) is None:
            raise KernelLibraryError("linear: the output given does not fit")
        self._linear(x, weight, bias, EPILOGUES[activation], out, None)
        return out

    def linear_qkv(self, x, weight, bias, n_head, n_kv_head, head_dim, cache, slots, out_dtype):
        """The fused q/k/v projection; new keys and values also go to their cache rows (inside
        the projection kernel where it can, else with the page-write kernel)."""
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=self.device)
        sink = None
        if cache is not None and cache.writes:
            self._want(slots, torch.int32, "slot_mapping", 1)
            sink = (cache, slots, n_head, n_kv_head, head_dim)
        stored = self._linear(x, weight, bias, EPILOGUES["none"], out, None, kv_sink=sink)
        if sink is not None and not stored:
            self.kv_store(out, n_head, n_kv_head, head_dim, cache, slots)
        return out

    def linear_residual(self, x, weight, bias, residual32):
        self._want(residual32, torch.float32, "residual", 2)
        if residual32.shape != (x.shape[0], weight.shape[0]):
            raise KernelLibraryError("linear_residual: residual has the wrong shape")
        self._linear(x, weight, bias, EPILOGUES["residual"], None, residual32)

    # ---- the whole feed-forward in one kernel (small batches) ---------------------------------------
    FUSED_MLP_ROWS = 16

    def _residual_ring(self, residual32):
        """Two more buffers like ``residual32`` that take turns with it as the residual stream
        (see ``mlp_residual``): ``(next, spare)``, ``next`` all zeros.  They are remembered by the
        tensor that currently holds the stream, so a chain of calls in one step allocates and
        zeroes once."""
        entry = self._ring
        if entry is not None and entry[0] is residual32:
            return entry[1], entry[2]
        nxt = torch.empty_like(residual32)
        spare = torch.empty_like(residual32)
        self._run(self.lib.mg_zero_fill(_ptr(nxt), nxt.numel() * 4, self._stream()), "zero fill")
        return nxt, spare

    def _packed_proj(self, weight):
        """The second matrix of a feed-forward, [C, F], copied once into the order in which the
        fused kernel's lanes read it (``mg_mlp_pack_elements`` in mlp_fused.cu): a layout change
        made when a matrix is first seen, not a computation of the step."""
        key = weight.data_ptr()
        hit = self._packed.get(key)
        if hit is not None and hit[0] is weight:
            return hit[1]
        c, f = weight.shape
        groups = (f + 15) // 16
        padded = weight
        if groups * 16 != f:
            padded = torch.zeros((c, groups * 16), dtype=weight.dtype, device=weight.device)
            padded[:, :f] = weight
        packed = padded.view(c // 8, 8, groups, 4, 4).permute(2, 0, 1, 3, 4).contiguous()
        assert packed.numel() == self.lib.mg_mlp_pack_elements(c, f)
        self._packed[key] = (weight, packed)
        return packed

    def mlp_residual(self, y, fc_weight, fc_bias, proj_weight, proj_bias, activation, residual32, act_dtype):
        """``residual32 + proj(act(fc(y)))``.  Returns the tensor that holds the sum: ``residual32``
        itself (added in place by two projection kernels), or, where the whole feed-forward runs as
        one kernel (bfloat16, up to 16 tokens, ``y`` a deferred LayerNorm of ``residual32``),
        another tensor: that kernel cannot write where its CTAs still read, so the residual
        stream moves between three buffers that take turns."""
        deferred = y if isinstance(y, DeferredNorm) else None
        m = residual32.shape[0]
        if (self.use_fused_mlp and deferred is not None and deferred.rows is None and deferred.x32 is residual32
                and activation in ("gelu_tanh", "relu_sq") and fc_weight.dtype == torch.bfloat16 and act_dtype == torch.bfloat16
                and deferred.dtype == torch.bfloat16 and 0 < m <= self.FUSED_MLP_ROWS
                and residual32.shape[1] <= self.lib.mg_mlp_fused_max_width() and residual32.shape[1] % 8 == 0
                and fc_weight.shape[0] % 8 == 0):
            self._want(residual32, torch.float32, "residual", 2)
            self._want(fc_weight, torch.bfloat16, "fc weight", 2)
            self._want(proj_weight, torch.bfloat16, "proj weight", 2)
            c, f = residual32.shape[1], fc_weight.shape[0]
            if fc_weight.shape != (f, c) or proj_weight.shape != (c, f):
                raise KernelLibraryError("feed-forward: the two matrices do not fit the width")
            for b, n, name in ((fc_bias, f, "fc bias"), (proj_bias, c, "proj bias")):
                if b is not None and self._want(b, torch.float32, name, 1).numel() != n:
                    raise KernelLibraryError(f"feed-forward: {name} has the wrong length")
            nxt, spare = self._residual_ring(residual32)
            code = self.lib.mg_mlp_fused(_ptr(residual32), _ptr(nxt), _ptr(spare), _ptr(deferred.gain),
                                         _ptr(deferred.shift), deferred.eps, _ptr(fc_weight), _ptr(fc_bias),
                                         _ptr(self._packed_proj(proj_weight)), _ptr(proj_bias), m, c, f,
                                         1 if activation == "relu_sq" else 0, self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "feed-forward (fused)")
                self._ring = (nxt, spare, residual32)          # nxt holds the stream; spare is zero
                return nxt
            self._ring = None
        h = self.linear(y, fc_weight, fc_bias, activation, act_dtype)
        self.linear_residual(h, proj_weight, proj_bias, residual32)
        return residual32

    def scale_(self, x32, scale: float):
        """``x32 *= scale`` in place (32-bit)."""
        self._want(x32, torch.float32, "scale input")
        self._run(self.lib.mg_scale(_ptr(x32), x32.numel(), float(scale), self._stream()), "scale")
        return x32

    def logits(self, y, tok_emb, greedy_out=None, vocab_limit=None, scale=1.0):
        """Logits in 32-bit, times ``scale``.  With ``greedy_out`` (int32 ``[rows]``): the argmax of
        every row (ids at or above ``vocab_limit`` excluded) is left there as well; returns
        ``(logits, taken)`` then, ``taken`` False if the projection that ran cannot take it on its
        way (a scale that is not positive would turn the order around: then it never does)."""
        if greedy_out is None:
            out = self.linear(y, tok_emb, None, "none", torch.float32)
            return out if scale == 1.0 else self.scale_(out, scale)
        self._ids_out(greedy_out, y.shape[0])
        out = torch.empty((y.shape[0], tok_emb.shape[0]), dtype=torch.float32, device=self.device)
        self.greedy_taken = False
        self._linear(y, tok_emb, None, EPILOGUES["none"], out, None,
                     greedy=(greedy_out, vocab_limit) if scale > 0 else None)
        if scale != 1.0:
            self.scale_(out, scale)
        return out, self.greedy_taken

    # ---- attention ------------------------------------------------------------------------------
    def kv_store(self, qkv, n_head, n_kv_head, head_dim, cache, slot_mapping):
        self._want(qkv, cache.k_pages.dtype, "qkv", 2)
        self._want(slot_mapping, torch.int32, "slot_mapping", 1)
        self._want(cache.k_pages, None, "k_pages", 4)
        self._want(cache.v_pages, cache.k_pages.dtype, "v_pages", 4)
        if qkv.shape[1] != (n_head + 2 * n_kv_head) * head_dim:
            raise KernelLibraryError("kv_store: qkv width does not match the head sizes")
        if tuple(cache.k_pages.shape[1:]) != (n_kv_head, cache.page_tokens, head_dim):
            raise KernelLibraryError("kv_store: page storage does not match the head sizes")
        self._run(self.lib.mg_kv_store(_ptr(qkv), _ptr(slot_mapping), _ptr(cache.k_pages),
                                   _ptr(cache.v_pages), qkv.shape[0], n_head, n_kv_head, head_dim,
                                   cache.page_tokens, cache.k_pages.shape[0], self._is_bf16(qkv),
                                   self._stream()), "kv_store")

    SPLIT_HEAD_DIMS = (16, 32, 64, 128, 256)

    PREFILL_TC_HEAD_DIMS = (64,)

    def _attention_tiles_name(self, n_head: int) -> str:
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # work items of the tiled kernel that run at once, per head (two CTAs per SM)
        return f"attention_tiles/{max(1, 2 * self._sm_count // n_head)}"

    def plan_prompt_attention(self, batch, plan, n_head, n_kv_head, head_dim) -> None:
        """Host half of the tiled prompt attention: the work list of a step (``attention_plan``),
        added to ``plan`` under a name that layers of equal head count share.  Nothing is planned
        for steps that the tiled kernel does not serve."""
        if (batch.decode_only or batch.act_dtype != torch.bfloat16 or not self.use_tensor_cores
                or not self.use_prefill_tc or head_dim not in self.PREFILL_TC_HEAD_DIMS):
            return
        name = self._attention_tiles_name(n_head)
        if name not in plan.arrays:
            import numpy as np

            slots = int(name.rsplit("/", 1)[1])
            # (steps of a shape that came before take their list from a small table)
            key = (tuple(batch.q_len), tuple(batch.ctx_before), slots)
            work = self._tile_lists.get(key)
            if work is None:
                work = np.asarray(query_tiles(batch.q_len, batch.ctx_before, slots), dtype=np.int32).reshape(-1, 5)
                if len(self._tile_lists) >= 64:
                    self._tile_lists.pop(next(iter(self._tile_lists)))
                self._tile_lists[key] = work
            plan.arrays[name] = work.copy()                  # (the table's copy stays as it is)
            plan.signature.append(("attention_merge", batch.max_ctx_after > KEY_CHUNK))

    def paged_attention(self, qkv, n_head, n_kv_head, head_dim, scale, cache, ctx):
        self._want(qkv, cache.k_pages.dtype, "qkv", 2)
        table = self._want(ctx.block_tables[cache.group], torch.int32, "block_table", 2)
        n = qkv.shape[0]
        out = torch.empty((n, n_head * head_dim), dtype=qkv.dtype, device=self.device)
        window = int(cache.window or 0)
        if (qkv.dtype == torch.bfloat16 and getattr(ctx, "decode_only", False)
                and head_dim in self.SPLIT_HEAD_DIMS and self.use_split_attention):
            # single query tokens: split along the keys; the last block of each row merges
            splits = self.lib.mg_attention_split_count(int(ctx.max_ctx_after), window, head_dim)
            floats = self.lib.mg_attention_split_scratch_floats(n, n_head, head_dim, splits)
            scratch = torch.empty((floats,), dtype=torch.float32, device=self.device)
            self._run(self.lib.mg_paged_attention_split(
                _ptr(qkv), _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(table),
                _ptr(ctx.token_request), _ptr(ctx.positions), _ptr(out), _ptr(scratch),
                _ptr(self._counters(n * n_head)), n, n_head, n_kv_head, head_dim, cache.page_tokens,
                table.shape[1], window, splits, float(scale), cache.k_pages.shape[0], table.shape[0],
                _ptr(self.status), self._stream()),
                "paged_attention (split)")
            # a grid of several waves merges in a kernel of its own
            self.launches += self.lib.mg_attention_split_launches(n, n_head, n_kv_head, splits) - 1
            return out
        work = getattr(ctx, "extra", {}).get(self._attention_tiles_name(n_head))
        if (qkv.dtype == torch.bfloat16 and work is not None and work.shape[0] > 0
                and self.use_tensor_cores and self.use_prefill_tc
                and head_dim in self.PREFILL_TC_HEAD_DIMS):
            # portions of prompts: query tiles of 128 on the tensor cores
            self._want(work, torch.int32, "attention tiles", 2)
            # tiles cut along the keys leave partial rows in scratch; the part that finishes last merges them
            merge = int(ctx.max_ctx_after > KEY_CHUNK)
            partial = counters = None
            if merge:
                floats = self.lib.mg_attention_prefill_scratch_floats(work.shape[0], n_head)
                partial = torch.empty((floats,), dtype=torch.float32, device=self.device)
                counters = self._counters(work.shape[0] * n_head)
            code = self.lib.mg_attention_prefill_tc(
                _ptr(qkv), _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(work), _ptr(table),
                _ptr(ctx.positions), _ptr(out), _ptr(partial), _ptr(counters), merge, work.shape[0], n, n_head,
                n_kv_head, head_dim,
                cache.page_tokens, cache.k_pages.shape[0], table.shape[1], window, float(scale),
                table.shape[0], 0, None, 0, _ptr(self.status), self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "paged_attention (prefill, tensor cores)")
                return out
        self._run(self.lib.mg_paged_attention_generic(
            _ptr(qkv), _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(table),
            _ptr(ctx.token_request), _ptr(ctx.positions), _ptr(out), n, n_head, n_kv_head, head_dim,
            cache.page_tokens, table.shape[1], window, float(scale), cache.k_pages.shape[0], table.shape[0],
            self._is_bf16(qkv), self._stream()), "paged_attention")
        return out

    def head_prepare(self, proj, n_head, n_kv_head, head_dim, v_dim, q_off, k_off, v_off, unit_norm, eps,
                     cache, slots, positions, v_other=None, blend=None, q_gain=None, k_gain=None):
        """Between a fused projection and the attention, in one kernel (``q_gain`` / ``k_gain``: 32-bit gains of
        ``head_dim`` numbers on the unit-RMS query and key heads): query and key heads of
        ``proj`` rows divided by their root mean square (``unit_norm``; queries in place), values
        blended with ``v_other`` (a 2-D view whose rows' first columns are the other values of the
        same tokens; ``blend`` a 32-bit scalar on the device), keys and values written to the cache
        rows ``slots`` (``cache`` None or read-only: nothing is written)."""
        self._want(proj, None, "projection rows", 2)
        is_bf16 = self._is_bf16(proj)
        args_other = [None, 0, None]
        if v_other is not None:
            if (v_other.dtype != proj.dtype or v_other.dim() != 2 or v_other.stride(1) != 1
                    or v_other.shape[0] != proj.shape[0] or v_other.shape[1] < n_kv_head * v_dim):
                raise KernelLibraryError("head_prepare: the other values do not fit the rows")
            self._want(blend, torch.float32, "blend weight")
            args_other = [_ptr(v_other), v_other.stride(0), _ptr(blend)]
        pages = [None, None, None, 0, 0]
        if cache is not None and cache.writes:
            self._want(slots, torch.int32, "slot_mapping", 1)
            self._want(cache.k_pages, proj.dtype, "k_pages", 4)
            self._want(cache.v_pages, proj.dtype, "v_pages", 4)
            if (tuple(cache.k_pages.shape[1:]) != (n_kv_head, cache.page_tokens, head_dim)
                    or tuple(cache.v_pages.shape[1:]) != (n_kv_head, cache.page_tokens, v_dim)):
                raise KernelLibraryError("head_prepare: page storage does not match the head sizes")
            pages = [_ptr(slots), _ptr(cache.k_pages), _ptr(cache.v_pages), cache.page_tokens, cache.k_pages.shape[0]]
        self._run(self.lib.mg_head_prepare(
            _ptr(proj), proj.shape[1], proj.shape[0], n_head, n_kv_head, head_dim, v_dim, q_off, k_off, v_off,
            1 if unit_norm else 0, float(eps), *args_other, pages[0], _ptr(positions), pages[1], pages[2],
            pages[3], pages[4], is_bf16, _ptr(self._gain(q_gain, head_dim)), _ptr(self._gain(k_gain, head_dim)),
            self._stream()), "head_prepare")

    def _gain(self, gain, size):
        if gain is not None and self._want(gain, torch.float32, "head gain", 1).numel() != size:
            raise KernelLibraryError("head_prepare: a gain does not match the head size")
        return gain

    def paged_attention_general(self, q, n_head, n_kv_head, head_dim, v_dim, scale, cache, ctx, gate=None,
                                slopes=None, block=None, softcap=None, sinks=None):
        """Causal attention of ``q`` (a 2-D tensor whose rows' first ``n_head * head_dim`` columns
        are the queries) over the pages, keys of size ``head_dim`` and values of size ``v_dim``;
        with ``gate`` (a 2-D view, ``n_head * v_dim`` columns) the output is multiplied by the
        logistic function of the gate values.  ``slopes`` (32-bit, one per head): ``slope * (i - j)``
        is taken off the score of query ``i`` and key ``j``; ``block``: a query sees only the keys
        of its own block of that many positions; ``softcap``: a score ``s`` (scale included) becomes
        ``softcap * tanh(s / softcap)``; ``sinks`` (32-bit, one per head): ``exp(sink)`` is added to the
        softmax's denominator.  A cache whose values live in its key rows is read that way.  Returns
        ``[tokens, n_head * v_dim]``."""
        if sinks is not None and self._want(sinks, torch.float32, "sinks", 1).numel() != n_head:
            raise KernelLibraryError("attention: one sink per head")
        softcap = float(softcap or 0.0)
        in_keys = bool(getattr(cache, "values_in_keys", False))
        plain = softcap == 0.0 and sinks is None and not in_keys      # what the tensor-core kernels take
        if slopes is not None and self._want(slopes, torch.float32, "slopes", 1).numel() != n_head:
            raise KernelLibraryError("attention: one slope per head")
        block = int(block or 0)
        biased = slopes is not None or block > 0
        self._want(q, cache.k_pages.dtype, "queries", 2)
        table = self._want(ctx.block_tables[cache.group], torch.int32, "block_table", 2)
        n = q.shape[0]
        if gate is not None and (gate.dtype != q.dtype or gate.dim() != 2 or gate.stride(1) != 1
                                 or gate.shape != (n, n_head * v_dim)):
            raise KernelLibraryError("attention: the gate does not fit the heads")
        out = torch.empty((n, n_head * v_dim), dtype=q.dtype, device=self.device)
        work = getattr(ctx, "extra", {}).get(self._attention_tiles_name(n_head)) if hasattr(ctx, "extra") else None
        if (q.dtype == torch.bfloat16 and work is not None and work.shape[0] > 0 and head_dim == v_dim and not biased
                and plain and head_dim in self.PREFILL_TC_HEAD_DIMS and self.use_tensor_cores and self.use_prefill_tc
                and not getattr(ctx, "decode_only", False)):
            # equal key and value sizes that the tcgen05 prompt attention takes: its tiles, with the
            # rows' own width and the gate in its epilogue
            merge = int(ctx.max_ctx_after > KEY_CHUNK)
            partial = counters = None
            if merge:
                floats = self.lib.mg_attention_prefill_scratch_floats(work.shape[0], n_head)
                partial = torch.empty((floats,), dtype=torch.float32, device=self.device)
                counters = self._counters(work.shape[0] * n_head)
            code = self.lib.mg_attention_prefill_tc(
                _ptr(q), _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(work), _ptr(table), _ptr(ctx.positions),
                _ptr(out), _ptr(partial), _ptr(counters), merge, work.shape[0], n, n_head, n_kv_head, head_dim,
                cache.page_tokens, cache.k_pages.shape[0], table.shape[1], int(cache.window or 0), float(scale),
                table.shape[0], q.shape[1], _ptr(gate), gate.stride(0) if gate is not None else 0,
                _ptr(self.status), self._stream())
            if code != library.UNSUPPORTED:
                self._run(code, "paged_attention (prefill, tensor cores)")
                return out
        if q.dtype == torch.bfloat16 and self.use_tensor_cores and self.use_mma_attention:
            # bfloat16: tiles of (token, head) rows on the warp-level tensor cores; single tokens
            # with their keys cut into ranges that a second kernel merges
            single = bool(getattr(ctx, "decode_only", False))
            q_len = getattr(ctx, "host_q_len", None)
            group = n_head // n_kv_head
            args = None
            if single:
                keys = self.lib.mg_attention_mma_split_keys(int(ctx.max_ctx_after))
                # (with a block mask a token's keys begin at its block: ranges are counted from the key
                # block of 64 that holds the block's first position)
                span = int(ctx.max_ctx_after) if block <= 0 else min(int(ctx.max_ctx_after), block + 64)
                splits = max(1, -(-span // keys))
                floats = self.lib.mg_attention_mma_scratch_floats(n, n_head, v_dim, splits)
                scratch = torch.empty((floats,), dtype=torch.float32, device=self.device)
                # (measured at batch 8, context 2,048: the ranges merged by a second kernel, 0.273 ms a
                # step; by the last CTA of each token and key/value head, 0.283 ms)
                counters = self._counters(n * n_kv_head) if self.merge_ranges_in_last_cta else None
                args = [_ptr(scratch), _ptr(counters), 1, 0, 1, splits, keys]
            elif q_len and group <= 64 and getattr(ctx, "req_q_start", None) is not None:
                tile = max(1, 64 // group)
                args = [None, None, 0, sum(-(-int(t) // tile) for t in q_len), tile, 0, 0]
            if args is not None:
                code = self.lib.mg_attention_mma(
                    _ptr(q), q.shape[1], _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(table), _ptr(ctx.token_request),
                    _ptr(ctx.positions), _ptr(getattr(ctx, "req_q_start", None)), _ptr(getattr(ctx, "req_q_len", None)),
                    _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out), args[0], args[1], n, table.shape[0],
                    n_head, n_kv_head, head_dim, v_dim, cache.page_tokens, table.shape[1], int(cache.window or 0),
                    float(scale), cache.k_pages.shape[0], *args[2:], _ptr(slopes), block, softcap, _ptr(sinks),
                    head_dim if in_keys else 0, self._stream())
                if code != library.UNSUPPORTED:
                    self._run(code, "paged_attention (tensor cores, general)")
                    if single and args[1] is None:
                        self.launches += 1                       # the merge of the ranges as a kernel of its own
                    return out
        if q.dtype == torch.bfloat16 and self.use_tensor_cores and self.use_mma_attention and in_keys and not biased:
            # rows too wide for that kernel's registers (cached latents of several hundred features): tiles of 32
            # (token, head) rows whose queries wait in shared memory
            single = bool(getattr(ctx, "decode_only", False))
            q_len = getattr(ctx, "host_q_len", None)
            group = n_head // n_kv_head
            args = None
            if single:
                keys = self.lib.mg_attention_mma_split_keys(int(ctx.max_ctx_after))
                splits = max(1, -(-int(ctx.max_ctx_after) // keys))
                floats = self.lib.mg_attention_mma_scratch_floats(n, n_head, v_dim, splits)
                scratch = torch.empty((floats,), dtype=torch.float32, device=self.device)
                args = [_ptr(scratch), 1, 0, splits, keys]
            elif q_len and getattr(ctx, "req_q_start", None) is not None:
                args = [None, 0, sum(self.lib.mg_attention_wide_tiles(int(t), group) for t in q_len), 0, 0]
            if args is not None:
                code = self.lib.mg_attention_wide(
                    _ptr(q), q.shape[1], _ptr(cache.k_pages), _ptr(table), _ptr(ctx.token_request), _ptr(ctx.positions),
                    _ptr(getattr(ctx, "req_q_start", None)), _ptr(getattr(ctx, "req_q_len", None)), _ptr(gate),
                    gate.stride(0) if gate is not None else 0, _ptr(out), args[0], n, table.shape[0], n_head, n_kv_head,
                    head_dim, v_dim, cache.page_tokens, table.shape[1], int(cache.window or 0), float(scale),
                    cache.k_pages.shape[0], *args[1:], softcap, _ptr(sinks), self._stream())
                if code != library.UNSUPPORTED:
                    self._run(code, "paged_attention (tensor cores, wide rows)")
                    if single:
                        self.launches += 1                       # the merge of the ranges
                    return out
        self._run(self.lib.mg_paged_attention_general(
            _ptr(q), q.shape[1], _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(table), _ptr(ctx.token_request),
            _ptr(ctx.positions), _ptr(out), n, n_head, n_kv_head, head_dim, v_dim, _ptr(gate),
            gate.stride(0) if gate is not None else 0, cache.page_tokens, table.shape[1], int(cache.window or 0),
            float(scale), cache.k_pages.shape[0], table.shape[0], self._is_bf16(q), _ptr(slopes), block,
            softcap, _ptr(sinks), head_dim if in_keys else 0, self._stream()), "paged_attention (general)")
        return out

    # ---- several residual streams ------------------------------------------------------------------
    def streams_spread(self, x32, streams):
        """``[streams, tokens, width]``, every stream a copy of ``x32``."""
        self._want(x32, torch.float32, "stream", 2)
        out = torch.empty((int(streams), *x32.shape), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_streams_spread(_ptr(x32), _ptr(out), int(streams), x32.numel(), self._stream()), "streams (spread)")
        return out

    def streams_read(self, streams32, weights, want_zeros=False):
        """``u = sum_s weights[s] * streams32[s]``; with ``want_zeros`` also a buffer of zeros of u's shape
        (returns ``(u, zeros)``), into which a sublayer can add its output."""
        self._want(streams32, torch.float32, "streams", 3)
        if self._want(weights, torch.float32, "stream weights", 1).numel() != streams32.shape[0]:
            raise KernelLibraryError("streams: one weight per stream")
        u = torch.empty(streams32.shape[1:], dtype=torch.float32, device=self.device)
        zeros = torch.empty_like(u) if want_zeros else None
        self._run(self.lib.mg_streams_read(_ptr(streams32), _ptr(weights), _ptr(u), _ptr(zeros), streams32.shape[0],
                                           u.numel(), self._stream()), "streams (read)")
        return (u, zeros) if want_zeros else u

    def streams_sum(self, streams32):
        hit = self._packed.get(("stream ones", streams32.shape[0]))
        if hit is None:
            hit = self._packed[("stream ones", streams32.shape[0])] = torch.ones(streams32.shape[0], dtype=torch.float32,
                                                                                device=self.device)
        return self.streams_read(streams32, hit)

    def streams_write(self, streams32, mix, weights, y32, next_read=None):
        """In place: ``streams32[t] = sum_s mix[s, t] * streams32[s] + weights[t] * y32`` for all t at once.  With
        ``next_read`` (the read weights of the sublayer that follows) returns ``(u, zeros)`` as ``streams_read`` of
        the new streams would."""
        self._want(streams32, torch.float32, "streams", 3)
        self._want(y32, torch.float32, "sublayer output", 2)
        s = streams32.shape[0]
        if (self._want(mix, torch.float32, "stream mix", 2).shape != (s, s) or y32.shape != streams32.shape[1:]
                or self._want(weights, torch.float32, "stream weights", 1).numel() != s):
            raise KernelLibraryError("streams: shapes do not fit")
        u = zeros = None
        if next_read is not None:
            if self._want(next_read, torch.float32, "stream weights", 1).numel() != s:
                raise KernelLibraryError("streams: one weight per stream")
            u, zeros = torch.empty_like(y32), torch.empty_like(y32)
        self._run(self.lib.mg_streams_write(_ptr(streams32), _ptr(mix), _ptr(weights), _ptr(y32), _ptr(next_read), _ptr(u),
                                            _ptr(zeros), s, y32.numel(), self._stream()), "streams (write)")
        return (u, zeros) if next_read is not None else None

    # ---- queries and keys that turn with the position ---------------------------------------------------
    def qk_norm_rotary(self, proj, n_head, n_kv_head, head_dim, v_dim, q_off, k_off, v_off, norm, eps, rot_dims, freq,
                       cache, slots, positions, q_gain=None, k_gain=None, v_unit_norm=False, v_freq=None):
        """Between a fused projection and the attention: optionally one RMS norm over all query features of a
        token and one over all key features (gains of those whole sizes), then the first ``rot_dims`` features of
        every query and key head turned by ``position * freq[i]`` (``freq``: 32-bit ``[rot_dims / 2]``); queries in
        place, keys and values to the cache rows ``slots`` (``cache`` None or read-only: nothing is written).
        ``v_unit_norm``: every value head is divided by its root mean square (``eps``, no gain) on its way to the cache;
        ``v_freq`` (32-bit ``[v_dim / 2]``): all features of every value head then turn by ``position * v_freq[m]``,
        feature ``m`` paired with ``m + v_dim / 2``."""
        self._want(proj, None, "projection rows", 2)
        if v_freq is not None and (v_dim % 2 or self._want(v_freq, torch.float32, "value frequencies", 1).numel() != v_dim // 2):
            raise KernelLibraryError("qk_norm_rotary: one frequency per pair of value features")
        self._want(positions, torch.int32, "positions", 1)
        if rot_dims and self._want(freq, torch.float32, "rotary frequencies", 1).numel() != rot_dims // 2:
            raise KernelLibraryError("qk_norm_rotary: one frequency per pair of turning features")
        for gain, size in ((q_gain, n_head * head_dim), (k_gain, n_kv_head * head_dim)):
            if gain is not None and self._want(gain, torch.float32, "norm gain", 1).numel() != size:
                raise KernelLibraryError("qk_norm_rotary: a gain does not match its projection")
        pages = [None, None, None, 0, 0]
        if cache is not None and cache.writes:
            self._want(slots, torch.int32, "slot_mapping", 1)
            self._want(cache.k_pages, proj.dtype, "k_pages", 4)
            self._want(cache.v_pages, proj.dtype, "v_pages", 4)
            if (tuple(cache.k_pages.shape[1:]) != (n_kv_head, cache.page_tokens, head_dim)
                    or tuple(cache.v_pages.shape[1:]) != (n_kv_head, cache.page_tokens, v_dim)):
                raise KernelLibraryError("qk_norm_rotary: page storage does not match the head sizes")
            pages = [_ptr(slots), _ptr(cache.k_pages), _ptr(cache.v_pages), cache.page_tokens, cache.k_pages.shape[0]]
        self._run(self.lib.mg_qk_norm_rotary(
            _ptr(proj), proj.shape[1], proj.shape[0], n_head, n_kv_head, head_dim, v_dim, q_off, k_off, v_off,
            1 if norm else 0, float(eps), _ptr(q_gain), _ptr(k_gain), int(rot_dims), _ptr(freq), _ptr(positions), pages[0],
            pages[1], pages[2], pages[3], pages[4], self._is_bf16(proj), 1 if v_unit_norm else 0, float(eps), _ptr(v_freq),
            self._stream()), "qk_norm_rotary")

    def rotate_heads(self, heads, n_head, v_dim, freq, positions, sign=-1.0):
        """Every head of ``heads`` ``[tokens, n_head * v_dim]`` turned in place by ``sign * position * freq[m]``, feature
        ``m`` paired with ``m + v_dim / 2`` (``sign`` -1: back into the frame of the token's own position)."""
        self._want(heads, None, "heads", 2)
        self._want(positions, torch.int32, "positions", 1)
        if (heads.shape[1] != n_head * v_dim or v_dim % 2 or positions.numel() != heads.shape[0]
                or self._want(freq, torch.float32, "frequencies", 1).numel() != v_dim // 2):
            raise KernelLibraryError("rotate_heads: shapes do not fit")
        self._run(self.lib.mg_rotate_heads(_ptr(heads), heads.shape[0], n_head, v_dim, _ptr(freq), _ptr(positions),
                                           float(sign), self._is_bf16(heads), self._stream()), "rotate_heads")
        return heads

    # ---- recurrences over single features, blends with the token before ------------------------------------
    def gated_recurrence(self, ctx, pre, z_off, u_off, g_off, width, state, state_offset, out_dtype):
        """``s <- (1 - sigmoid(z)) s + sigmoid(z) cand(u)`` feature by feature over every request's tokens, from and to
        the requests' state slots (``width`` numbers from ``state_offset``); ``cand(u) = u + 1/2`` for ``u >= 0`` and
        ``sigmoid(u)`` below.  ``pre``: 32-bit rows with z, u and an output gate g at the three offsets.  Returns
        ``s * silu(g)`` ``[tokens, width]`` in ``out_dtype``.  A bfloat16 step whose longest portion has
        ``RECURRENCE_RANGE_MIN_TOKENS`` tokens or more runs the form whose warps share a request's tokens; 32-bit
        steps always run token by token (one fixed order of sums whatever the cut)."""
        self._want(pre, torch.float32, "pre-activations", 2)
        self._want(state, torch.float32, "state slots", 2)
        if state_offset < 0 or state_offset + width > state.shape[1]:
            raise KernelLibraryError("gated_recurrence: the state slots are too small")
        n = pre.shape[0]
        out = torch.empty((n, width), dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_gated_recurrence(
            _ptr(pre), pre.shape[1], z_off, u_off, g_off, _ptr(ctx.req_q_start), _ptr(ctx.req_q_len), _ptr(ctx.req_ctx_before),
            _ptr(ctx.req_state_slot), state.data_ptr() + 4 * int(state_offset), state.shape[1], _ptr(out),
            ctx.req_q_start.numel(), n, width, state.shape[0], self._is_bf16(out),
            1 if (out_dtype == torch.bfloat16 and self.use_recurrence_ranges
                  and int(getattr(ctx, "max_q_len", 0)) >= self.RECURRENCE_RANGE_MIN_TOKENS) else 0,
            self._stream()), "gated_recurrence")
        return out

    RECURRENCE_RANGE_MIN_TOKENS = 128

    def token_shift_mix(self, ctx, x, mu, state):
        """``out[s] = x_t + (x_(t-1) - x_t) * mu[s]`` for every row of ``mu`` ``[mixes, width]`` (32-bit): ``[mixes, tokens,
        width]`` in x's type.  The row before a request's first row of the step comes from the head of its state slot
        (zeros for a sequence's first token); ``conv_state_update`` with two taps leaves the step's last row there."""
        self._want(x, None, "rows", 2)
        self._want(mu, torch.float32, "blend weights", 2)
        self._want(state, torch.float32, "state slots", 2)
        n, width = x.shape
        if mu.shape[1] != width or state.shape[1] < width:
            raise KernelLibraryError("token_shift_mix: shapes do not fit")
        out = torch.empty((mu.shape[0], n, width), dtype=x.dtype, device=self.device)
        self._run(self.lib.mg_token_shift_mix(
            _ptr(x), _ptr(mu), _ptr(ctx.token_request), _ptr(ctx.positions), _ptr(ctx.req_q_start), _ptr(ctx.req_ctx_before),
            _ptr(ctx.req_state_slot), _ptr(state), state.shape[1], _ptr(out), n, width, mu.shape[0], ctx.req_q_start.numel(),
            state.shape[0], self._is_bf16(x), self._stream()), "token_shift_mix")
        return out

    # ---- sums into the residual stream ------------------------------------------------------------------------
    def zeros32(self, rows, width, ctx=None, index=0):
        """A zeroed 32-bit buffer a sublayer can add its output into.  With ``ctx``: buffer number ``index`` of the
        forward pass that ``ctx`` belongs to, made and zeroed at its first use; whoever takes it leaves it as zeros
        again (``rmsnorm_add`` and ``scaled_sum_`` with ``clear``), so one zero fill serves a whole pass."""
        shared = getattr(ctx, "shared", None)
        key = ("zeros32", rows, width, index)
        if shared is not None and key in shared:
            return shared[key]
        out = torch.empty((rows, width), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_zero_fill(_ptr(out), out.numel() * 4, self._stream()), "zero fill")
        if shared is not None:
            shared[key] = out
        return out

    def rmsnorm_add(self, residual32, y32, weight, eps, offset=0.0, other32=None, scale=1.0, other_scale=1.0, clear=False):
        """``residual32 += rms_norm(scale * y32 [+ other_scale * other32]) * (offset + weight)``, in place, 32-bit.
        ``clear``: ``y32`` (and ``other32``) are left as zeros, ready for the next sublayer to add into."""
        self._want(residual32, torch.float32, "residual", 2)
        self._want(y32, torch.float32, "sublayer output", 2)
        self._want(weight, torch.float32, "norm weight", 1)
        if other32 is not None:
            self._want(other32, torch.float32, "second sublayer output", 2)
        if y32.shape != residual32.shape or weight.numel() != residual32.shape[1] or (other32 is not None and other32.shape != y32.shape):
            raise KernelLibraryError("rmsnorm_add: shapes do not fit")
        self._run(self.lib.mg_rmsnorm_add(_ptr(residual32), _ptr(y32), float(scale), _ptr(other32), float(other_scale),
                                          _ptr(weight), residual32.shape[0], residual32.shape[1], float(eps), float(offset),
                                          1 if clear else 0, self._stream()), "rmsnorm_add")
        return residual32

    def add_rows(self, x32, rows32, vector):
        """``x32 += rows32 + vector`` in place (``rows32`` None: the vector alone; ``vector``: ``[width]`` 32-bit)."""
        self._want(x32, torch.float32, "stream", 2)
        self._want(vector, torch.float32, "vector", 1)
        if rows32 is not None and self._want(rows32, torch.float32, "rows", 2).shape != x32.shape:
            raise KernelLibraryError("add_rows: shapes do not fit")
        if vector.numel() != x32.shape[1]:
            raise KernelLibraryError("add_rows: the vector does not match the width")
        self._run(self.lib.mg_add_rows(_ptr(x32), _ptr(rows32), _ptr(vector), x32.numel(), x32.shape[1], self._stream()),
                  "add_rows")
        return x32

    def scaled_sum_(self, x32, a32, scale_a, b32, scale_b, clear=False):
        """``x32 += scale_a * a32 + scale_b * b32`` in place, 32-bit.  ``clear``: ``a32`` and ``b32`` are left as zeros."""
        for name, t in (("sum", x32), ("first term", a32), ("second term", b32)):
            self._want(t, torch.float32, name, 2)
        if a32.shape != x32.shape or b32.shape != x32.shape:
            raise KernelLibraryError("scaled_sum: shapes do not fit")
        self._run(self.lib.mg_scaled_sum(_ptr(x32), _ptr(a32), float(scale_a), _ptr(b32), float(scale_b), x32.numel(),
                                         1 if clear else 0, self._stream()), "scaled_sum")
        return x32

    def softcap_(self, x32, cap: float):
        """``x32 <- cap * tanh(x32 / cap)`` in place (32-bit)."""
        self._want(x32, torch.float32, "softcap input")
        self._run(self.lib.mg_softcap(_ptr(x32), x32.numel(), float(cap), self._stream()), "softcap")
        return x32

    def cast(self, x32, out_dtype):
        """32-bit rows in ``out_dtype`` (the tensor itself if that is 32-bit)."""
        self._want(x32, torch.float32, "rows")
        if out_dtype == torch.float32:
            return x32
        out = torch.empty(x32.shape, dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_cast_rows(_ptr(x32), _ptr(out), x32.numel(), 0, self._is_bf16(out), self._stream()), "cast")
        return out

    def tanh_cast(self, x32, out_dtype):
        """``tanh(x32)`` in ``out_dtype`` (the tanh itself in 32-bit)."""
        self._want(x32, torch.float32, "rows")
        out = torch.empty(x32.shape, dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_cast_rows(_ptr(x32), _ptr(out), x32.numel(), 1, self._is_bf16(out), self._stream()), "tanh")
        return out

    def token_side_residual(self, ctx, residual32, gate_weight, proj_weight, norm_weight, table, offset, eps, act_dtype):
        """``g = gelu_tanh(gate_weight x) * table[token, offset : offset + dim]``, ``y = proj_weight g``,
        ``residual32 += y / sqrt(mean(y^2) + eps) * norm_weight`` with ``x`` the rows of ``residual32`` themselves, in
        place: two projections with the gate between and the norm behind them.  ``x`` and ``g`` are rounded to
        ``act_dtype`` on their way into the products; everything else is 32-bit.  (The whole of it as one kernel, a
        CTA a token, was measured for steps of few tokens: 37 us a layer where these kernels take 14 inside a
        replayed graph, because a token's CTA pulls both matrices through one SM.)"""
        self._want(residual32, torch.float32, "residual", 2)
        self._want(gate_weight, act_dtype, "gate matrix", 2)
        self._want(proj_weight, act_dtype, "projection matrix", 2)
        n, width = residual32.shape
        dim = gate_weight.shape[0]
        if gate_weight.shape != (dim, width) or proj_weight.shape != (width, dim):
            raise KernelLibraryError("token_side: shapes do not fit")
        gate = self.linear(self.cast(residual32, act_dtype), gate_weight, None, "none", torch.float32)
        gated = self.token_gate(ctx, gate, table, offset, act_dtype)
        y = self.linear(gated, proj_weight, None, "none", torch.float32)
        return self.rmsnorm_add(residual32, y, norm_weight, eps)

    def token_gate(self, ctx, gate32, table, offset, out_dtype):
        """``gelu_tanh(gate32) * table[token, offset : offset + dim]``, ``dim`` the width of ``gate32``, in ``out_dtype``
        (the table's type).  Tokens that the step before sampled are taken from its ids, as the embedding does."""
        self._want(gate32, torch.float32, "gate", 2)
        self._want(table, out_dtype, "token table", 2)
        n, dim = gate32.shape
        if offset < 0 or offset + dim > table.shape[1] or ctx.token_ids.numel() != n:
            raise KernelLibraryError("token_gate: shapes do not fit")
        source, previous = getattr(ctx, "token_source", None), getattr(ctx, "fed_ids", None)
        out = torch.empty((n, dim), dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_token_gate(_ptr(gate32), _ptr(ctx.token_ids), _ptr(ctx.positions), _ptr(source),
                                         _ptr(previous) if source is not None else None, _ptr(table), table.shape[1], int(offset),
                                         _ptr(out), n, dim, table.shape[0], previous.numel() if source is not None else 0,
                                         self._is_bf16(table), self._is_bf16(out), self._stream()), "token_gate")
        return out

    def latent_prepare(self, proj, n_head, q_off, q_dim, rot_dim, low_off, rank, gain, eps, freq, cache, slots, positions):
        """For an attention over cached latents.  Returns ``q`` ``[tokens, n_head * (rank + rot_dim)]`` whose last
        ``rot_dim`` features per head are the turned last ``rot_dim`` features of the query heads in ``proj``
        (``n_head x (q_dim + rot_dim)`` from ``q_off``); the first ``rank`` per head are left for ``head_linear``.
        With a writable ``cache``: the ``rank`` numbers of ``proj`` from ``low_off``, RMS-normed with ``gain``, and the
        ``rot_dim`` behind them, turned, go to the token's cache row."""
        self._want(proj, None, "projection rows", 2)
        self._want(positions, torch.int32, "positions", 1)
        if rot_dim and self._want(freq, torch.float32, "rotary frequencies", 1).numel() != rot_dim // 2:
            raise KernelLibraryError("latent_prepare: one frequency per pair of turning features")
        pages = [None, None, None, 0, 0]
        if cache is not None and cache.writes:
            self._want(slots, torch.int32, "slot_mapping", 1)
            self._want(cache.k_pages, proj.dtype, "k_pages", 4)
            self._want(gain, torch.float32, "latent gain", 1)
            if tuple(cache.k_pages.shape[1:]) != (1, cache.page_tokens, rank + rot_dim) or gain.numel() != rank:
                raise KernelLibraryError("latent_prepare: page storage does not match the latent's size")
            separate = None if getattr(cache, "values_in_keys", False) else self._want(cache.v_pages, proj.dtype, "v_pages", 4)
            if separate is not None and tuple(separate.shape[1:]) != (1, cache.page_tokens, rank):
                raise KernelLibraryError("latent_prepare: value pages do not match the latent's size")
            pages = [_ptr(slots), _ptr(cache.k_pages), _ptr(separate), cache.page_tokens, cache.k_pages.shape[0]]
        q = torch.empty((proj.shape[0], n_head * (rank + rot_dim)), dtype=proj.dtype, device=self.device)
        self._run(self.lib.mg_latent_prepare(
            _ptr(proj), proj.shape[1], proj.shape[0], n_head, q_off, q_dim, int(rot_dim), low_off, rank, _ptr(gain),
            float(eps), _ptr(freq), _ptr(q), _ptr(positions), pages[0], pages[1], pages[2], pages[3], pages[4],
            self._is_bf16(proj), self._stream()), "latent_prepare")
        return q

    def head_linear(self, x, x_off, x_head, weight, rows_are_inputs, n_head, n_in, n_out, gate=None, out=None, out_off=0,
                    out_head=None):
        """One small matrix per head: ``out[n, h, j] = sum_i x[n, h, i] * W_h[j, i]`` with ``weight``
        ``[n_head * n_out, n_in]``, or, with ``rows_are_inputs``, ``sum_i x[n, h, i] * W_h[i, j]`` with ``weight``
        ``[n_head * n_in, n_out]``.  Head h's inputs are the columns ``x_off + h * x_head ..`` of ``x``; its outputs go
        to the columns ``out_off + h * out_head ..`` of ``out`` (a new ``[tokens, n_head * n_out]`` tensor unless
        given).  ``gate`` (a 2-D view, ``n_head * n_out`` columns): the outputs times its logistic function."""
        self._want(x, weight.dtype, "head inputs", 2)
        self._want(weight, None, "head matrices", 2)
        if weight.shape != ((n_head * n_in, n_out) if rows_are_inputs else (n_head * n_out, n_in)):
            raise KernelLibraryError("head_linear: the matrices do not fit the heads")
        n = x.shape[0]
        if gate is not None and (gate.dtype != x.dtype or gate.dim() != 2 or gate.stride(1) != 1
                                 or gate.shape != (n, n_head * n_out)):
            raise KernelLibraryError("head_linear: the gate does not fit the heads")
        if out is None:
            out, out_off, out_head = torch.empty((n, n_head * n_out), dtype=x.dtype, device=self.device), 0, n_out
        else:
            self._want(out, x.dtype, "head outputs", 2)
            out_head = n_out if out_head is None else out_head
            if out.shape[0] != n:
                raise KernelLibraryError("head_linear: one output row per token")
        self._run(self.lib.mg_head_linear(
            _ptr(x), x.shape[1], x_off, x_head, _ptr(weight), 1 if rows_are_inputs else 0, _ptr(gate),
            gate.stride(0) if gate is not None else 0, _ptr(out), out.shape[1], out_off, out_head, n, n_head, n_in, n_out,
            self._is_bf16(x), self._stream()), "head_linear")
        return out

    # ---- around the scan of a state-space mixer ---------------------------------------------------------
    def causal_conv_silu(self, ctx, x, x_off, channels, taps, bias, state):
        """``silu(bias + causal convolution)`` per channel over every request's tokens (``taps``: 32-bit
        ``[channels, n]``, the last column weighs the current token); the ``n - 1`` inputs before a step's first
        token come from the head of the request's state slot.  Returns ``[tokens, channels]`` in x's type."""
        self._want(x, None, "convolution inputs", 2)
        self._want(taps, torch.float32, "taps", 2)
        self._want(state, torch.float32, "state slots", 2)
        if taps.shape[0] != channels or (bias is not None and self._want(bias, torch.float32, "bias", 1).numel() != channels):
            raise KernelLibraryError("causal_conv: taps and bias do not fit the channels")
        out = torch.empty((x.shape[0], channels), dtype=x.dtype, device=self.device)
        self._run(self.lib.mg_causal_conv_silu(
            _ptr(x), x.shape[1], x_off, _ptr(taps), _ptr(bias), _ptr(ctx.token_request), _ptr(ctx.positions),
            _ptr(ctx.req_q_start), _ptr(ctx.req_ctx_before), _ptr(ctx.req_state_slot), _ptr(state), state.shape[1], _ptr(out),
            x.shape[0], channels, taps.shape[1], ctx.req_q_start.numel(), state.shape[0], self._is_bf16(x), self._stream()),
            "causal_conv")
        return out

    def conv_state_update(self, ctx, x, x_off, channels, n_taps, state):
        """After ``causal_conv_silu`` of the same step: the last ``n_taps - 1`` inputs of every request's sequence go
        to the head of its state slot."""
        if n_taps <= 1:
            return
        self._run(self.lib.mg_conv_state_update(
            _ptr(x), x.shape[1], x_off, _ptr(ctx.req_q_start), _ptr(ctx.req_q_len), _ptr(ctx.req_ctx_before),
            _ptr(ctx.req_state_slot), _ptr(state), state.shape[1], ctx.req_q_start.numel(), channels, int(n_taps),
            state.shape[0], self._is_bf16(x), self._stream()), "conv_state_update")

    def gated_group_norm(self, out32, gate, gain, parts, eps, out_dtype, positions=None):
        """``rms_norm(out32 * silu(gate))`` taken over ``parts`` equal parts of a row apart, times ``gain``."""
        self._want(out32, torch.float32, "scan output", 2)
        self._want(gain, torch.float32, "norm gain", 1)
        n, width = out32.shape
        if (gate.dtype != out_dtype or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape != (n, width)
                or gain.numel() != width or width % parts):
            raise KernelLibraryError("gated_group_norm: shapes do not fit")
        out = torch.empty((n, width), dtype=out_dtype, device=self.device)
        self._run(self.lib.mg_gated_group_norm(_ptr(out32), _ptr(gate), gate.stride(0), _ptr(gain), _ptr(positions), _ptr(out),
                                               n, width, int(parts), float(eps), self._is_bf16(out), self._stream()),
                  "gated_group_norm")
        return out

    # ---- routed experts ---------------------------------------------------------------------------
    def moe_route(self, y, router_weight, gate_weight, positions, top):
        """Router of a feed-forward of experts: returns (ids [tokens, top] int32, weights [tokens,
        top] 32-bit, gate [tokens] 32-bit or None): the ``top`` largest of ``router_weight @ y``
        with the softmax over them, and the logistic function of ``gate_weight . y``."""
        self._want(y, None, "router input", 2)
        self._want(router_weight, torch.float32, "router weight", 2)
        n, width = y.shape
        experts = router_weight.shape[0]
        if router_weight.shape[1] != width or not 0 < top <= experts:
            raise KernelLibraryError("moe_route: shapes do not fit")
        ids = torch.empty((n, top), dtype=torch.int32, device=self.device)
        weights = torch.empty((n, top), dtype=torch.float32, device=self.device)
        gate = None
        if gate_weight is not None:
            self._want(gate_weight, torch.float32, "gate weight")
            if gate_weight.numel() != width:
                raise KernelLibraryError("moe_route: the gate's weights do not fit the width")
            gate = torch.empty((n,), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_moe_route(_ptr(y), _ptr(router_weight), _ptr(gate_weight), _ptr(positions), _ptr(ids),
                                        _ptr(weights), _ptr(gate), n, width, experts, top, self._is_bf16(y),
                                        self._stream()), "moe route")
        return ids, weights, gate

    def moe_route_scored(self, y, router_weight, gate_weight, positions, top, scoring, correction, groups, scale):
        """As ``moe_route`` with a score per expert: ``scoring`` ``"sigmoid"`` (weights ``scale * sigmoid(z)``
        of the chosen, not renormalised) or ``"softmax_top"`` (``scale`` times the softmax over the chosen
        logits); ``correction`` (32-bit, one per expert, or None) is added for the choice only; ``groups``
        ``(count, keep)`` or None: only experts of the ``keep`` best of ``count`` equal groups of neighbours
        (a group's score: the sum of its two largest choice scores) can be chosen."""
        self._want(y, None, "router input", 2)
        self._want(router_weight, torch.float32, "router weight", 2)
        n, width = y.shape
        experts = router_weight.shape[0]
        if router_weight.shape[1] != width or not 0 < top <= experts:
            raise KernelLibraryError("moe_route: shapes do not fit")
        if correction is not None and self._want(correction, torch.float32, "correction", 1).numel() != experts:
            raise KernelLibraryError("moe_route: one correction per expert")
        if scoring not in ("sigmoid", "softmax_top"):
            raise KernelLibraryError(f"moe_route: scoring {scoring!r}")
        count, keep = groups if groups is not None else (0, 0)
        ids = torch.empty((n, top), dtype=torch.int32, device=self.device)
        weights = torch.empty((n, top), dtype=torch.float32, device=self.device)
        gate = None
        if gate_weight is not None:
            self._want(gate_weight, torch.float32, "gate weight")
            if gate_weight.numel() != width:
                raise KernelLibraryError("moe_route: the gate's weights do not fit the width")
            gate = torch.empty((n,), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_moe_route_scored(_ptr(y), _ptr(router_weight), _ptr(gate_weight), _ptr(correction),
                                               _ptr(positions), _ptr(ids), _ptr(weights), _ptr(gate), n, width, experts,
                                               top, 1 if scoring == "sigmoid" else 0, int(count), int(keep), float(scale),
                                               self._is_bf16(y), self._stream()), "moe route (scored)")
        return ids, weights, gate

    def moe_experts_residual(self, y, ids, weights, w_in, w_out, residual32, activation="silu", limit=0.0):
        """``residual32[t] += sum_k weights[t, k] * expert(ids[t, k])(y[t])`` with expert e as
        ``w_out[e] @ (silu(w_in[e][:F] @ y) * (w_in[e][F:] @ y))``; ``w_in`` [E, 2F, C], ``w_out``
        [E, C, F].  Tokens are grouped by expert on the device; the host never learns the counts."""
        self._want(y, w_in.dtype, "expert input", 2)
        self._want(w_in, None, "expert matrices (in)", 3)
        self._want(w_out, w_in.dtype, "expert matrices (out)", 3)
        self._want(residual32, torch.float32, "residual", 2)
        n, width = y.shape
        experts, two_f, _ = w_in.shape
        inner, top = two_f // 2, ids.shape[1]
        if (w_in.shape != (experts, 2 * inner, width) or w_out.shape != (experts, width, inner)
                or ids.shape[0] != n or weights.shape != ids.shape or residual32.shape != (n, width)):
            raise KernelLibraryError("moe_experts: shapes do not fit")
        entries = n * top
        is_bf16 = self._is_bf16(y)
        act = GATED_ACTIVATIONS[activation]
        offsets = torch.empty((experts + 1,), dtype=torch.int32, device=self.device)
        slot_entry = torch.empty((entries,), dtype=torch.int32, device=self.device)
        entry_slot = torch.empty((entries,), dtype=torch.int32, device=self.device)
        self._run(self.lib.mg_moe_group(_ptr(ids), entries, experts, _ptr(offsets), _ptr(slot_entry), _ptr(entry_slot),
                                        self._stream()), "moe group")
        hidden = torch.empty((entries, inner), dtype=y.dtype, device=self.device)
        self._run(self.lib.mg_moe_gemm(_ptr(y), width, _ptr(w_in), _ptr(offsets), _ptr(slot_entry), top, None,
                                       _ptr(hidden), experts, n, inner, width, n, 1, is_bf16, act, float(limit),
                                       self._stream()),
                  "moe experts (in)")
        out = torch.empty((entries, width), dtype=torch.float32, device=self.device)
        self._run(self.lib.mg_moe_gemm(_ptr(hidden), inner, _ptr(w_out), _ptr(offsets), _ptr(slot_entry), top,
                                       _ptr(weights), _ptr(out), experts, n, width, inner, entries, 0, is_bf16, 0, 0.0,
                                       self._stream()), "moe experts (out)")
        self._run(self.lib.mg_moe_combine(_ptr(out), _ptr(entry_slot), top, _ptr(residual32), n, width, entries,
                                          self._stream()), "moe combine")

    def glu(self, gate_up, row_scale=None, activation="silu", limit=0.0):
        """``silu(gate_up[:, :F]) * gate_up[:, F:]``, each row times ``row_scale`` (32-bit ``[rows]``)
        if given; the result has the input's dtype.  ``activation``: ``silu``, ``gelu_tanh`` (in place of
        silu) or ``clamped_swish`` (``g * sigmoid(1.702 g) * (u + 1)`` with ``g = min(gate, limit)``,
        ``u = clamp(up, -limit, limit)``)."""
        self._want(gate_up, None, "gate and up features", 2)
        rows, two_f = gate_up.shape
        if two_f % 2:
            raise KernelLibraryError("glu: an odd number of columns")
        if row_scale is not None and self._want(row_scale, torch.float32, "row scale", 1).numel() != rows:
            raise KernelLibraryError("glu: one scale per row")
        out = torch.empty((rows, two_f // 2), dtype=gate_up.dtype, device=self.device)
        self._run(self.lib.mg_glu(_ptr(gate_up), _ptr(row_scale), _ptr(out), rows, two_f // 2, self._is_bf16(gate_up),
                                  GATED_ACTIVATIONS[activation], float(limit), self._stream()), "glu")
        return out

    # ---- sampling -------------------------------------------------------------------------------
    def _ids_out(self, out, rows):
        if out is None:
            return torch.empty((rows,), dtype=torch.int32, device=self.device)
        self._want(out, torch.int32, "ids", 1)
        if out.numel() != rows:
            raise KernelLibraryError(f"ids: room for {out.numel()} rows, {rows} wanted")
        return out

    def argmax(self, logits, vocab_limit=None, out=None):
        self._want(logits, torch.float32, "logits", 2)
        rows, vocab = logits.shape
        out = self._ids_out(out, rows)
        if vocab >= 8192 and rows <= 512:
            # few rows of a wide vocabulary: many blocks per row, then a merge
            parts = self.lib.mg_argmax_parts(vocab)
            scratch_v = torch.empty((rows * parts,), dtype=torch.float32, device=self.device)
            scratch_i = torch.empty((rows * parts,), dtype=torch.int32, device=self.device)
            self._run(self.lib.mg_argmax_wide(_ptr(logits), _ptr(out), _ptr(scratch_v),
                                          _ptr(scratch_i), rows, vocab, int(vocab_limit or 0),
                                          self._stream()), "argmax (wide)")
            self.launches += 1
            return out
        self._run(self.lib.mg_argmax(_ptr(logits), _ptr(out), rows, vocab,
                                 int(vocab_limit or 0), self._stream()), "argmax")
        return out

    def sample(self, logits, temperature, top_k, top_p, seed_lo, seed_hi, counter, vocab_limit=None,
               out=None):
        """One draw per row.  temperature float32 [rows]; top_k int32 [rows] or None (<= 0: off);
        top_p float32 [rows] or None (>= 1: off); seed_lo, seed_hi, counter: int32 [rows] holding
        the 32-bit words of each row's seed and the number of its draw."""
        self._want(logits, torch.float32, "logits", 2)
        rows = logits.shape[0]
        self._want(temperature, torch.float32, "temperature", 1)
        for name, t in (("top_k", top_k), ("seed_lo", seed_lo), ("seed_hi", seed_hi),
                        ("counter", counter)):
            if t is not None:
                self._want(t, torch.int32, name, 1)
        if top_p is not None:
            self._want(top_p, torch.float32, "top_p", 1)
        for t in (temperature, top_k, top_p, seed_lo, seed_hi, counter):
            if t is not None and t.numel() != rows:
                raise KernelLibraryError("sample: per-row parameters do not match the rows")
        out = self._ids_out(out, rows)
        self._run(self.lib.mg_sample(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                 _ptr(seed_lo), _ptr(seed_hi), _ptr(counter), _ptr(out), rows,
                                 logits.shape[1], int(vocab_limit or 0), self._stream()), "sample")
        return out


_default = {}


def default_ops(device="cuda:0") -> CudaOps:
    key = str(torch.device(device))
    if key not in _default:
        _default[key] = CudaOps(device)
    return _default[key]
