"""Python faces of the kernel entry points: tensors in, launches on the current stream.

Each function checks device, dtype, contiguity and sizes of what it is given (a kernel never sees
a pointer it could misread) and raises ``KernelError`` with the library's message when the library
refuses a size. Nothing here computes on the host.
"""
from __future__ import annotations

from typing import Optional

import torch

from .library import KernelError, check, lib

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype} (float32 and bfloat16 only)") from None


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process (each wrapper call launches one)."""
    return _launches


def count_launches(n: int) -> None:
    """Adjusts the count for kernels that run from a replayed CUDA graph (or were only captured)."""
    global _launches
    _launches += n


_scoped_stream: Optional[int] = None


class on_current_stream:
    """Within this block every kernel goes to the stream that is current at its entry: the handle is
    looked up once instead of at every launch (a few microseconds each, a third of a millisecond of a
    step that launches 150 kernels). Blocks nest (a graph capture inside a step has its own stream)."""

    def __enter__(self):
        global _scoped_stream
        self._outer = _scoped_stream
        _scoped_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._outer
        return False


def _stream() -> int:
    global _launches
    _launches += 1
    return _scoped_stream if _scoped_stream is not None else torch.cuda.current_stream().cuda_stream


class Program:
    """A recorded sequence of this library's launches (csrc/program.cu): ``run()`` repeats it on the
    current stream with one call into the library. It holds raw addresses and sizes, so it is valid
    only while every buffer it was recorded with is."""

    def __init__(self, handle: int, launches: int):
        self._handle = handle
        self.launches = launches

    def run(self) -> None:
        global _launches
        stream = _scoped_stream if _scoped_stream is not None else torch.cuda.current_stream().cuda_stream
        check(lib().gi_program_run(self._handle, stream), "program")
        _launches += self.launches

    def __len__(self) -> int:
        return int(lib().gi_program_size(self._handle))

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            try:
                lib().gi_program_free(handle)
            except Exception:       # interpreter shutdown
                pass


class record:
    """``with record() as r: ...`` runs the block's kernel calls as usual and records them;
    ``r.program`` repeats them afterwards. Recordings do not nest."""

    program: Optional[Program] = None

    def __enter__(self):
        check(lib().gi_program_begin(), "program")
        self._before = _launches
        return self

    def __exit__(self, exc_type, exc, tb):
        handle = lib().gi_program_end()
        if exc_type is None:
            self.program = Program(handle, _launches - self._before)
        elif handle:
            lib().gi_program_free(handle)
        return False


def _dev(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t: Optional[torch.Tensor], name: str, dtype: torch.dtype) -> int:
    return 0 if t is None else _dev(t, name, dtype)


def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
          feedback: Optional[torch.Tensor] = None) -> None:
    """out[t, :] = table[tokens[t], :] * scale, widened to 32-bit. A negative tokens[t] = -(k + 1)
    stands for feedback[k], a token id that a sampling kernel left on the device."""
    T, D = out.shape
    if table.shape[1] != D or tokens.numel() != T:
        raise KernelError("embed: shapes of table, tokens and out do not agree")
    check(lib().gi_embed(_dev(table, "table"), dtype_code(table.dtype), _dev(tokens, "tokens", torch.int32),
                         _opt(feedback, "feedback", torch.int32), _dev(out, "out", torch.float32), T, D, float(scale),
                         _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = weight * (x[row_r, :] / sqrt(mean(x^2) + eps)); ``rows`` gathers rows of x."""
    n, D = out.shape
    if x.shape[1] != D or weight.numel() != D:
        raise KernelError("rmsnorm: shapes of x, weight and out do not agree")
    if rows is None and x.shape[0] < n:
        raise KernelError("rmsnorm: x has fewer rows than out")
    if rows is not None and rows.numel() != n:
        raise KernelError("rmsnorm: rows and out do not agree")
    check(lib().gi_rmsnorm(_dev(x, "x", torch.float32), _opt(rows, "rows", torch.int32),
                           _dev(weight, "weight", torch.float32), _dev(out, "out"), dtype_code(out.dtype),
                           n, D, float(eps), _stream()), "rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError("swiglu: gate_up must be [T, 2I] for out [T, I]")
    check(lib().gi_swiglu(_dev(gate_up, "gate_up", torch.float32), _dev(out, "out"), dtype_code(out.dtype), T, I,
                          _stream()), "swiglu")


def rope_store(qkv: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, block_tables: torch.Tensor,
               cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], interleaved: bool,
               q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
               num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, write_kv: bool = True) -> None:
    """Rotates query and key heads of ``qkv`` [T, (H+2Hkv)*hd] by the rows of the cos/sin table at
    each token's position, writes queries to ``q_out`` [T, H*hd] and keys/values into the token's
    row of the paged cache [pages, Hkv, page_size, hd]."""
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("rope_store: qkv width does not match the head counts")
    if q_out.shape != (T, num_heads * head_dim):
        raise KernelError("rope_store: q_out must be [T, H*hd]")
    if k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype:
        raise KernelError("rope_store: q_out and the cache must have one dtype")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("rope_store: the cache must be [pages, Hkv, page_size, hd]")
    rot_half = 0 if cos is None else cos.shape[1]
    if cos is not None and (sin is None or sin.shape != cos.shape):
        raise KernelError("rope_store: cos and sin tables must have one shape")
    check(lib().gi_rope_store(
        _dev(qkv, "qkv", torch.float32), _dev(positions, "positions", torch.int32),
        _dev(row_req, "row_req", torch.int32), _dev(block_tables, "block_tables", torch.int32),
        block_tables.shape[1], _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), rot_half,
        int(interleaved), _dev(q_out, "q_out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
        dtype_code(q_out.dtype), T, num_heads, num_kv_heads, head_dim, page_size, int(write_kv), _stream()),
        "rope_store")


def copy_pages(cache: torch.Tensor, src: torch.Tensor, dst: torch.Tensor) -> None:
    """cache is [arrays, pages, ...]; copies page src[i] to page dst[i] in every array."""
    n_arrays = cache.shape[0]
    page_bytes = cache[0, 0].numel() * cache.element_size()
    array_stride = cache[0].numel() * cache.element_size()
    check(lib().gi_copy_pages(_dev(cache, "cache"), array_stride, n_arrays, page_bytes,
                              _dev(src, "src", torch.int32), _dev(dst, "dst", torch.int32), src.numel(),
                              _stream()), "copy_pages")


def attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                      row_req: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor,
                      num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                      window: Optional[int] = None) -> None:
    """Causal attention of every row of ``q`` [T, H*hd] over its request's pages."""
    T = q.shape[0]
    if q.shape != (T, num_heads * head_dim) or out.shape != q.shape or out.dtype != q.dtype:
        raise KernelError("attention: q and out must be [T, H*hd] of one dtype")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise KernelError("attention: q and the cache must have one dtype")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("attention: the cache must be [pages, Hkv, page_size, hd]")
    check(lib().gi_attention_generic(
        _dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), _dev(out, "out"), dtype_code(q.dtype),
        _dev(row_req, "row_req", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1], T, num_heads, num_kv_heads,
        head_dim, page_size, float(scale), int(window or 0), _stream()), "attention")


def attention_supported(head_dim: int) -> bool:
    """Whether any attention kernel of the library serves this head size (multiples of 16 up to 256)."""
    return bool(lib().gi_attention_generic_supported(head_dim))


def attention_fast_supported(head_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    """Whether the tensor-core attention kernels are built for this head size and grouping."""
    return bool(lib().gi_attention_fast_supported(head_dim, num_heads, num_kv_heads))


def attention_prefill_rows(page_size: int, head_dim: int) -> int:
    """Query rows (tokens x heads of one key/value group) per work item of the prefill kernel."""
    return int(lib().gi_attention_prefill_rows(page_size, head_dim))


def attention_chunk_keys() -> int:
    """Positions per chunk of the decode kernel's split over the context (a fixed length)."""
    return int(lib().gi_attention_chunk_keys())


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     rows: torch.Tensor, row_req: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor,
                     num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                     window: Optional[int], part_o: torch.Tensor, part_ml: torch.Tensor, max_chunks: int,
                     n_chunks: int) -> None:
    """Attention of single decoded tokens (bfloat16): ``rows`` lists their step rows; the context is
    split into fixed chunks whose partial results go through ``part_o`` / ``part_ml``."""
    n = rows.numel()
    if part_o.numel() < n * num_heads * max_chunks * head_dim or part_ml.numel() < n * num_heads * max_chunks * 2:
        raise KernelError("attention_decode: the workspace is too small")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("attention: the cache must be [pages, Hkv, page_size, hd]")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q and out must be [T, H*hd]")
    check(lib().gi_attention_decode(
        _dev(q, "q", torch.bfloat16), _dev(k_cache, "k_cache", torch.bfloat16), _dev(v_cache, "v_cache", torch.bfloat16),
        _dev(out, "out", torch.bfloat16), _dev(rows, "rows", torch.int32), n, _dev(row_req, "row_req", torch.int32),
        _dev(positions, "positions", torch.int32), _dev(block_tables, "block_tables", torch.int32),
        block_tables.shape[1], num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
        _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), max_chunks, n_chunks,
        k_cache.shape[0], _tc_state(q.device).status.data_ptr(), _stream()), "attention_decode")
    tma = page_size % 8 == 0 and (32 % page_size == 0 or page_size % 32 == 0)
    if n_chunks > 1 or not tma:
        count_launches(1)     # the kernel that merges the chunks (not needed when every context is one chunk)


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                      work: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor, num_heads: int,
                      num_kv_heads: int, head_dim: int, page_size: int, scale: float, window: Optional[int]) -> None:
    """Attention of prompt portions (bfloat16): ``work`` [n, 3] = (first step row of a tile, tokens
    in it (at most attention_prefill_rows() // group size), request index)."""
    if work.dim() != 2 or work.shape[1] != 3:
        raise KernelError("attention_prefill: work must be [n, 3]")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("attention: the cache must be [pages, Hkv, page_size, hd]")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q and out must be [T, H*hd]")
    check(lib().gi_attention_prefill(
        _dev(q, "q", torch.bfloat16), _dev(k_cache, "k_cache", torch.bfloat16), _dev(v_cache, "v_cache", torch.bfloat16),
        _dev(out, "out", torch.bfloat16), _dev(work, "work", torch.int32), work.shape[0],
        _dev(positions, "positions", torch.int32), _dev(block_tables, "block_tables", torch.int32),
        block_tables.shape[1], num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
        k_cache.shape[0], _tc_state(q.device).status.data_ptr(), _stream()), "attention_prefill")


def attention_prefill_tc_supported(head_dim: int, num_heads: int, num_kv_heads: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention serves this shape (head size 64 or 128, pages TMA can tile)."""
    return bool(lib().gi_attention_prefill_tc_supported(head_dim, num_heads, num_kv_heads, page_size))


def attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                         work: torch.Tensor, positions: torch.Tensor, block_tables: torch.Tensor, num_heads: int,
                         num_kv_heads: int, head_dim: int, page_size: int, scale: float, window: Optional[int]) -> None:
    """Attention of prompt portions on the tcgen05 tensor cores: ``work`` [n, 3] = (first step row of
    a tile, tokens in it (at most 128 // group size), request index)."""
    if work.dim() != 2 or work.shape[1] != 3:
        raise KernelError("attention_prefill_tc: work must be [n, 3]")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("attention: the cache must be [pages, Hkv, page_size, hd]")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q and out must be [T, H*hd]")
    check(lib().gi_attention_prefill_tc(
        _dev(q, "q", torch.bfloat16), _dev(k_cache, "k_cache", torch.bfloat16), _dev(v_cache, "v_cache", torch.bfloat16),
        _dev(out, "out", torch.bfloat16), _dev(work, "work", torch.int32), work.shape[0],
        _dev(positions, "positions", torch.int32), _dev(block_tables, "block_tables", torch.int32),
        block_tables.shape[1], num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
        k_cache.shape[0], _tc_state(q.device).status.data_ptr(), _stream()), "attention_prefill_tc")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out[M,N] (+)= a[M,K] @ w[N,K]^T with 32-bit fused multiply-adds on the CUDA cores."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm: shapes do not agree (a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)})")
    check(lib().gi_gemm_simt(_dev(a, "a"), dtype_code(a.dtype), _dev(w, "w"), dtype_code(w.dtype), _dev(out, "out"),
                             dtype_code(out.dtype), int(accumulate), M, N, K, K, K, N, _stream()), "gemm")


class _TensorCoreState:
    """Per-device buffers of the tensor-core matrix product: the workspace and tile counters of the
    split over K, and the status word in which a kernel records a wait that gave up."""

    WORKSPACE_FLOATS = 8 * 1024 * 1024
    COUNTERS = 4096

    def __init__(self, device: torch.device):
        self.device = device
        self._workspace = None
        self.counters = torch.zeros(self.COUNTERS, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    @property
    def workspace(self) -> torch.Tensor:
        if self._workspace is None:        # only products split over K need it (the 32-bit path never does)
            self._workspace = torch.empty(self.WORKSPACE_FLOATS, dtype=torch.float32, device=self.device)
        return self._workspace


_tc_states = {}


def _tc_state(device: torch.device) -> _TensorCoreState:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _tc_states:
        _tc_states[key] = _TensorCoreState(device)
    return _tc_states[key]


_B200_SMS = 148          # only for looking at plans on a machine without a device
_sm_count: Optional[int] = None


def sm_count() -> int:
    """Streaming multiprocessors of the device the kernels run on (asked once); the plans below
    size their grids by it. Without a device (plans examined on a CPU) the B200's count."""
    global _sm_count
    if _sm_count is None:
        if torch.cuda.is_available():
            _sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
        else:
            return _B200_SMS
    return _sm_count


# Many-token products on pairs of CTAs (tcgen05 cta_group::2): the two CTAs of a pair share a 256-row tile of
# tokens and each fetches half of the weights' tile, so an SM takes in 32 KB instead of 48 KB per 64 columns of K.
PAIRED_PRODUCTS = True


def _paired(M: int, block_q: int) -> int:
    return int(PAIRED_PRODUCTS and M > 128 and block_q == 256)


def _persistent_plan(M: int, N: int, K: int):
    block_q = 256 if N >= 256 else 128 if N > 64 else 64
    splits = 1
    if block_q >= 128 and N % 4 == 0:
        # few output tiles (a prompt portion of a few hundred tokens, a narrow matrix): K is cut as well
        # so that about as many work items as SMs exist, each with at least 8 steps of 64
        tiles = ((M + 127) // 128) * ((N + block_q - 1) // block_q)
        k_blocks = (K + 63) // 64
        splits = max(1, min(8, sm_count() // tiles, k_blocks // 8))
        if splits < 3 and k_blocks < 64:
            splits = 1           # measured: two ranges of a short K cost more (a second kernel adds them) than they save
    return False, block_q, splits


def gemm_tc_plan(M: int, N: int, K: int, accumulate: bool = False):
    """(swap, block_q, splits) for a product of these sizes; the choice depends on the sizes (and on whether the
    product is added into its output) only.
    Few tokens put the weights on the 128-row side (the tokens are the N of the MMA) and split K until
    the grid fills the GPU. Many tokens put the tokens on the 128-row side, one persistent CTA per SM,
    K cut into ranges when the output has few tiles. Between 65 and 128 tokens a narrow matrix with a long K (one
    that the first form would split) is faster in the second form, whose ranges are added up by a
    kernel of their own instead of by one CTA per tile (measured at the Llama-3.2-1B widths: the down product of
    128 tokens 30 -> 17 us); with a short K, token tiles of 32 (or, for a product that is stored, of 64) in the first
    form are faster still (the O product of 128 tokens 11.5 -> 8.6 us, [q; k; v] 12.3 -> 9.6 us; at the Llama-3.1-8B
    widths [q; k; v] 30.5 -> 17.6 us)."""
    if M <= 128:
        tiles, k_blocks = (N + 127) // 128, (K + 63) // 64
        if M > 64 and k_blocks <= 64:
            if tiles * ((M + 31) // 32) * 2 <= sm_count():
                return True, 32, 2 if k_blocks >= 8 else 1
            if not accumulate and tiles * ((M + 63) // 64) <= sm_count():
                return True, 64, 1
        swap, block_q, splits = _swap_plan(M, N, K)
        if M > 32 and N >= 256 and N % 4 == 0 and (splits >= 6 or (M > 64 and splits > 1)):
            return _persistent_plan(M, N, K)
        return swap, block_q, splits
    return _persistent_plan(M, N, K)


_STREAMING_SHARE = 0.75


def _swap_plan(M: int, N: int, K: int):
    block_q = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    tiles = (N + 127) // 128
    k_blocks = (K + 63) // 64
    if 32 < M <= 64 and 2 * tiles * 2 <= sm_count():
        # 33 to 64 tokens over a matrix of few row tiles: two tiles of 32 tokens, each with its own CTAs (the second reads the
        # weights from L2), so that what the 32-token form has applies: ranges of K added up in a cluster, residual values
        # and rotation tables requested early, rotation in the epilogue. Measured at the Llama-3.2-1B widths, 64 tokens:
        # the O product 11.1 -> 7.3 us, down 16.1 -> 12.3, [q; k; v] 10.1 -> 8.6 (and no rotation kernel after it).
        splits = 1
        while 2 * tiles * (splits + 1) <= sm_count() and k_blocks // (splits + 1) >= 4 and splits < 5:
            splits += 1
        return True, 32, splits
    # split K until about three quarters of the SMs stream weights (112 CTAs on a B200), keeping at least
    # 4 steps of 64 per CTA (measured on B200 at the Llama-3.2-1B widths: 4 splits for 24 tiles, 6..8 for 16, 1 for 128)
    streaming = int(sm_count() * _STREAMING_SHARE) + 1
    # (17 to 32 tokens: at most 5 ranges, whose partial tiles have a place of their own beside four stages; measured at the
    # Llama-3.2-1B widths, 32 tokens: the O product 9.9 -> 8.6 us, down 13.4 -> 12.8)
    most = 5 if block_q == 32 else 8
    splits = 1
    while tiles * (splits + 1) <= streaming and k_blocks // (splits + 1) >= 4 and splits < most:
        splits += 1
    return True, block_q, splits


_cluster_splits_cache = {}


def gemm_tc_cluster_splits(block_q: int, tiles: int, splits: int, tiled: bool = False) -> int:
    """The split count to run: the planned one, or up to two fewer if only then all the launch's
    clusters (one per tile, a CTA per split) are resident at once, which lets the splits be added up
    in shared memory instead of through global memory. A property of the device, asked once."""
    key = (block_q, tiles, splits, tiled)
    if key not in _cluster_splits_cache:
        chosen = None
        # first with the partial tiles in shared memory of their own (no split waits for another), then
        # in the first split's pipeline stages (it tells the others when they are free)
        # (the first only while it keeps three quarters of the planned splits: fewer CTAs streaming the
        # weights cost more than the wait)
        for sign in (-1, 1):
            for s in range(splits, max(1, splits - 3), -1):
                if sign < 0 and 4 * s < 3 * splits:
                    continue
                if chosen is None and s >= 2 and lib().gi_gemm_tc_cluster_capacity(block_q, sign * s, int(tiled)) >= tiles:
                    chosen = s
        _cluster_splits_cache[key] = chosen or splits
    return _cluster_splits_cache[key]


def tile_weight(w: torch.Tensor) -> torch.Tensor:
    """A copy of the bfloat16 matrix w [N, K] laid out as the few-token product reads it: tiles of
    128 rows x 64 columns in the order [row tile][column block], each tile 16 KB in the swizzled
    K-major layout of the tensor cores (row r at r * 128 bytes, its 16-byte pieces permuted by
    piece ^ (r % 8)), rows padded with zeros to a multiple of 128 and columns to a multiple of 128.
    One untiled bulk copy then brings two neighbouring tiles (32 KB) into shared memory, which a B200
    SM does at 1.5 times the rate of tiled TMA boxes, with half as many waits and commits."""
    N, K = w.shape
    Np, Kp = (N + 127) // 128 * 128, (K + 127) // 128 * 128
    wp = torch.zeros((Np, Kp), dtype=w.dtype, device=w.device)
    wp[:N, :K] = w
    t = wp.view(Np // 128, 128, Kp // 64, 8, 8).permute(0, 2, 1, 3, 4)          # [row tile, k block, row, piece, 8]
    r = torch.arange(128, device=w.device).view(128, 1)
    piece = torch.arange(8, device=w.device).view(1, 8)
    src = (piece ^ (r % 8)).view(1, 1, 128, 8, 1).expand(t.shape[0], t.shape[1], 128, 8, 8)
    return torch.gather(t, 3, src).contiguous().view(-1)        # place q of row r holds piece q ^ (r % 8)


_gemm_choice = {}      # (M, N, K, output dtype, tiled weights) -> (swap, block_q, splits, persistent): the sizes decide, once


# How much of the weights that a later product will stream a few-token product asks into L2 (measured on B200 at the
# Llama-3.2-1B widths: 16 to 24 MiB ahead of the [gate; up] product make a decode step 1 to 3 % faster, 48 MiB slower)
AHEAD_BYTES = 24 << 20


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False, plan=None,
            w_tiles: Optional[torch.Tensor] = None, ahead: Optional[torch.Tensor] = None) -> None:
    """out[M,N] (+)= a[M,K] @ w[N,K]^T on the tensor cores: bfloat16 operands, 32-bit accumulation,
    output 32-bit (optionally accumulated into) or bfloat16. K must be a multiple of 8. ``w_tiles``
    (tile_weight(w)) lets products of few tokens fetch the weights with bulk copies. ``ahead``: a tensor
    that a later kernel of the step streams (the tile-by-tile weights of the next large product); a product of few
    tokens asks its first AHEAD_BYTES into L2 while it runs, so that memory keeps streaming between the kernels."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm: shapes do not agree (a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)})")
    key = (M, N, K, out.dtype, w_tiles is not None, bool(accumulate)) if plan is None else None
    chosen = _gemm_choice.get(key) if key is not None else None
    if chosen is None:
        swap, block_q, splits = plan or gemm_tc_plan(M, N, K, bool(accumulate))
        persistent = not swap and out.dtype is torch.float32 and N % 4 == 0 and block_q >= 128
        if not swap and not persistent:
            if plan is None and M <= 128:
                swap, block_q, splits = _swap_plan(M, N, K)      # the persistent kernel cannot write this output
            else:
                splits = 1
        if plan is None and swap and splits > 1:
            splits = gemm_tc_cluster_splits(block_q, (N + 127) // 128 * ((M + block_q - 1) // block_q), splits,
                                            w_tiles is not None and block_q <= 128)
        chosen = (swap, block_q, splits, persistent)
        if key is not None:
            _gemm_choice[key] = chosen
    swap, block_q, splits, persistent = chosen
    st = _tc_state(a.device)
    if persistent:
        # many tokens, 32-bit output: the persistent kernel (epilogue overlapped, TMA stores)
        need = splits * ((M + 255) // 256 * 256) * N
        if splits > 1 and need > st.workspace.numel():
            splits = 1
        check(lib().gi_gemm_tc_persistent(_dev(a, "a", torch.bfloat16), _dev(w, "w", torch.bfloat16),
                                          _dev(out, "out", torch.float32), 1 if accumulate else 0, M, N, K, K, K, N,
                                          block_q, st.status.data_ptr(), splits, st.workspace.data_ptr() if splits > 1 else 0,
                                          st.workspace.numel() if splits > 1 else 0, _paired(M, block_q), _stream()), "gemm_tc")
        if splits > 1:
            count_launches(1)     # the kernel that adds the ranges up
        return
    check(lib().gi_gemm_tc(_dev(a, "a", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"),
                           dtype_code(out.dtype), int(accumulate), M, N, K, K, K, N, int(swap), block_q, splits,
                           st.workspace.data_ptr(), st.workspace.numel(), st.counters.data_ptr(), st.counters.numel(),
                           st.status.data_ptr(), _opt(w_tiles, "w_tiles", torch.bfloat16),
                           ahead.data_ptr() if ahead is not None and swap and M <= 32 else 0,
                           min(AHEAD_BYTES, ahead.numel() * ahead.element_size()) if ahead is not None else 0,
                           _stream()), "gemm_tc")


def gemm_swiglu_supported(M: int, I: int, K: int) -> bool:
    """The fused gate/up product needs many tokens (tokens on the 128-row side) and TMA-addressable rows."""
    return M > 128 and K % 8 == 0 and I % 8 == 0


def gemm_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] = silu(a @ w_gate^T) * (a @ w_up^T) as bfloat16, w_gate_up = [gate rows; up rows]
    [2I, K]: one tensor-core kernel whose epilogue applies the activation (the [M, 2I] intermediate
    never exists in memory)."""
    M, K = a.shape
    I = out.shape[1]
    if w_gate_up.shape != (2 * I, K) or out.shape[0] != M:
        raise KernelError("gemm_swiglu: shapes do not agree")
    st = _tc_state(a.device)
    check(lib().gi_gemm_tc_persistent(_dev(a, "a", torch.bfloat16), _dev(w_gate_up, "w_gate_up", torch.bfloat16),
                                      _dev(out, "out", torch.bfloat16), 2, M, I, K, K, K, I, 256,
                                      st.status.data_ptr(), 1, 0, 0, _paired(M, 256), _stream()), "gemm_swiglu")


_ROPE_FEW_TOKENS = 64      # up to here the few-token product (weights on the 128-row side, token tiles of at most 32) does
                           # the rotation: measured in whole decode steps, 2.4 % faster at 16 tokens (with 64-token tiles
                           # it was 1.7 % slower at 64 tokens)


def gemm_rope_store_supported(M: int, K: int, num_heads: int, num_kv_heads: int, head_dim: int,
                              cos: Optional[torch.Tensor], interleaved: bool) -> bool:
    """Whether the [q; k; v] product of M tokens can rotate and store in its own epilogue. Few tokens: the
    head size must divide 128 (both members of a pair in one tile of weight rows), any rotation. Many
    tokens: head sizes 32, 64, 128, whole heads rotated in the half-split pairing (or no rotation), and
    enough output tiles that K is not cut into ranges. Between the two, and otherwise, the product and
    the rope+store kernel run one after the other."""
    if K % 8:
        return False
    N = (num_heads + 2 * num_kv_heads) * head_dim
    if M <= 32 or (M <= _ROPE_FEW_TOKENS and _swap_plan(M, N, K)[1] == 32):      # token tiles of at most 32
        return 128 % head_dim == 0
    if head_dim not in (32, 64, 128) or not (cos is None or (not interleaved and 2 * cos.shape[1] == head_dim)):
        return False
    return M > 128 and _persistent_plan(M, N, K)[2] == 1


def gemm_rope_store(a: torch.Tensor, w_qkv: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor,
                    block_tables: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                    interleaved: bool, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, write_kv: bool = True,
                    w_tiles: Optional[torch.Tensor] = None) -> None:
    """``rope_store`` of ``a @ w_qkv^T`` in one tensor-core kernel: the product's epilogue rotates the
    query and key heads and writes queries to ``q_out`` and keys/values into the pages; the
    [T, (H+2Hkv)*hd] intermediate never exists in memory. All operands bfloat16."""
    M, K = a.shape
    N = (num_heads + 2 * num_kv_heads) * head_dim
    if w_qkv.shape != (N, K):
        raise KernelError("gemm_rope_store: the weight must be [(H+2Hkv)*hd, K]")
    if q_out.shape != (M, num_heads * head_dim):
        raise KernelError("gemm_rope_store: q_out must be [T, H*hd]")
    if k_cache.shape[1:] != (num_kv_heads, page_size, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError("gemm_rope_store: the cache must be [pages, Hkv, page_size, hd]")
    if cos is not None and (sin is None or sin.shape != cos.shape):
        raise KernelError("gemm_rope_store: cos and sin tables must have one shape")
    if not gemm_rope_store_supported(M, K, num_heads, num_kv_heads, head_dim, cos, interleaved):
        raise KernelError(f"gemm_rope_store: not built for {M} tokens, head size {head_dim} and this rotation")
    st = _tc_state(a.device)
    rope_args = (_dev(positions, "positions", torch.int32), _dev(row_req, "row_req", torch.int32),
                 _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1], _opt(cos, "cos", torch.float32),
                 _opt(sin, "sin", torch.float32), 0 if cos is None else cos.shape[1], int(interleaved),
                 _dev(q_out, "q_out", torch.bfloat16), _dev(k_cache, "k_cache", torch.bfloat16),
                 _dev(v_cache, "v_cache", torch.bfloat16), num_heads, num_kv_heads, head_dim, page_size, int(write_kv))
    if M <= _ROPE_FEW_TOKENS:
        _, block_q, splits = _swap_plan(M, N, K)
        if splits > 1:
            splits = gemm_tc_cluster_splits(block_q, (N + 127) // 128 * ((M + block_q - 1) // block_q), splits, w_tiles is not None)
        check(lib().gi_gemm_tc_rope(_dev(a, "a", torch.bfloat16), _dev(w_qkv, "w_qkv", torch.bfloat16), M, K, K, K, block_q,
                                    splits, st.workspace.data_ptr(), st.workspace.numel(), st.counters.data_ptr(),
                                    st.counters.numel(), st.status.data_ptr(), _opt(w_tiles, "w_tiles", torch.bfloat16),
                                    *rope_args, _stream()), "gemm_rope_store")
    else:
        check(lib().gi_gemm_tc_persistent_rope(_dev(a, "a", torch.bfloat16), _dev(w_qkv, "w_qkv", torch.bfloat16), M, K, K, K,
                                               *rope_args, st.status.data_ptr(), _paired(M, 256), _stream()), "gemm_rope_store")


def l2_streaming(weights: Optional[bool] = None, keys_values: Optional[bool] = None):
    """In steps of few tokens the weights of the matrix products and the keys and values of decode attention, which
    a step reads once, are loaded with the "evict first" L2 policy, so that they do not push out what the step's
    kernels read again soon. Sets either switch (None leaves it) and returns the old (weights, keys_values)."""
    old_w = bool(lib().gi_gemm_tc_set_stream_weights(1))
    lib().gi_gemm_tc_set_stream_weights(int(old_w if weights is None else weights))
    old_kv = bool(lib().gi_attention_set_stream_kv(1))
    lib().gi_attention_set_stream_kv(int(old_kv if keys_values is None else keys_values))
    return old_w, old_kv


def specialised_products(on: Optional[bool] = None) -> bool:
    """The forms of the few-token product that a decode step runs (rotating [q; k; v], added into the residual stream,
    stored unsplit; up to 16 tokens over tiled weights) have kernels of their own with nothing else compiled in;
    ``on`` False makes the kernel of every form run them too (same results). Returns the old setting."""
    old = bool(lib().gi_gemm_tc_set_specialised(1))
    lib().gi_gemm_tc_set_specialised(int(old if on is None else on))
    return old


def status_word(device: torch.device) -> torch.Tensor:
    """The device word [1] (int32) in which a kernel records a bounded wait that gave up (0 = none)."""
    return _tc_state(device).status


def gemm_tc_status(device: torch.device) -> int:
    """0 when no bounded wait of a tensor-core kernel ever gave up on this device (synchronises)."""
    import ctypes
    st = _tc_state(device)
    out = ctypes.c_int(0)
    check(lib().gi_gemm_tc_status(st.status.data_ptr(), torch.cuda.current_stream().cuda_stream, ctypes.byref(out)),
          "gemm_tc_status")
    return out.value


_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the largest logit of row r (the lowest index among equals)."""
    rows, V = logits.shape
    key = logits.device.index
    buf = _argmax_scratch.get(key)
    if buf is None or buf[0].numel() < rows * 32:
        n = max(rows, 64) * 32
        buf = (torch.empty(n, dtype=torch.float32, device=logits.device), torch.empty(n, dtype=torch.int32, device=logits.device))
        _argmax_scratch[key] = buf
    check(lib().gi_argmax(_dev(logits, "logits", torch.float32), rows, V, _dev(out, "out", torch.int32),
                          buf[0].data_ptr(), buf[1].data_ptr(), _stream()), "argmax")
    global _launches
    _launches += 1            # two kernels


def sample(logits: torch.Tensor, scratch: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
    rows, V = logits.shape
    if scratch.numel() < rows * V:
        raise KernelError("sample: scratch must hold rows x vocab floats")
    check(lib().gi_sample(_dev(logits, "logits", torch.float32), _dev(scratch, "scratch", torch.float32), rows, V,
                          _dev(temperature, "temperature", torch.float32), _dev(top_k, "top_k", torch.int32),
                          _dev(top_p, "top_p", torch.float32), _dev(uniform, "uniform", torch.float32),
                          _dev(out, "out", torch.int32), _stream()), "sample")
