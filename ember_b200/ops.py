"""Python face of the CUDA kernels: argument checks, then a ctypes call on the current stream.

There is no CPU fall-back and no library stand-in: every function raises ``KernelError`` if
its tensors are not on a CUDA device or if the compiled library is missing or refuses the
sizes.  Tensors are torch tensors used as typed device buffers.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
EPI_STORE, EPI_STORE_F32, EPI_ADD_F32, EPI_SILU_MUL = 0, 1, 2, 3
EPI_SUMS = 5      # tensor-core product of at most 128 tokens: the fp32 sums stay in the split-K scratch
EPI_RELU_MUL = 6  # the gated epilogue with relu: relu(c[2j]) * c[2j + 1]
EPI_GELU_MUL = 7  # ... with the tanh form of gelu: 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))) * c[2j + 1]
GATED_EPILOGUES = (EPI_SILU_MUL, EPI_RELU_MUL, EPI_GELU_MUL)
GATED_EPILOGUE_OF = {"silu": EPI_SILU_MUL, "relu": EPI_RELU_MUL, "gelu_tanh": EPI_GELU_MUL}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dt}")


def _check(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on a CUDA device only (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _p(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_libs = {}


def _lib(name: str):
    lib = _libs.get(name)
    if lib is None:
        try:
            lib = build.load(name)
        except (build.BuildError, OSError) as e:
            raise KernelError(f"the CUDA kernel library '{name}' is not available: {e}") from e
        _libs[name] = lib
    return lib


_launches = 0


def launch_count() -> int:
    """How many kernel-launching calls this process has made (each launches one or two kernels)."""
    return _launches


def add_launches(n: int) -> None:
    """A replayed CUDA graph launches the kernels that were captured into it."""
    global _launches
    _launches += n


def _call(lib, fn, *args):
    global _launches
    _launches += 1
    rc = fn(*args)
    if rc != 0:
        raise KernelError(lib.ember_last_error().decode("utf-8", "replace"))


# ------------------------------------------------------------------------------ elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None,
          stream: Optional[int] = None, prev_ids: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """out[t, :] = scale * float(table[tokens[t], :]).  With ``prev_ids`` (int32, device) a token -(r + 1) is
    read as prev_ids[r]: the id the sampler wrote there in the step before."""
    _check(tokens, "tokens", torch.int32)
    if prev_ids is not None:
        _check(prev_ids, "prev_ids", torch.int32)
    _check(table, "table")
    _check(out, "out", torch.float32)
    T, (V, H) = tokens.numel(), table.shape
    if out.shape[-1] != H or out.numel() < T * H:
        raise KernelError(f"embed: output {tuple(out.shape)} does not fit {T} rows of width {H}")
    lib = _lib("elementwise")
    _call(lib, lib.ember_embed, _p(tokens), _p(prev_ids), c_int(prev_ids.numel() if prev_ids is not None else 0),
          _p(table), c_int(dtype_code(table.dtype)), _p(out), c_int(T), c_int(H), c_int(V), c_float(scale), _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, n_rows: int,
            rows: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """out[r] = weight * x[rows[r] or r] * rsqrt(mean(x^2) + eps); x is fp32, statistics fp32."""
    _check(x, "x", torch.float32)
    _check(weight, "weight", torch.float32)
    _check(out, "out")
    H = x.shape[-1]
    if weight.numel() != H or out.shape[-1] != H or out.numel() < n_rows * H:
        raise KernelError(f"rmsnorm: width {H}, weight {tuple(weight.shape)}, out {tuple(out.shape)} for {n_rows} rows")
    if rows is not None:
        _check(rows, "rows", torch.int32)
    lib = _lib("elementwise")
    _call(lib, lib.ember_rmsnorm, _p(x), _p(rows), _p(weight), c_float(eps), _p(out), c_int(dtype_code(out.dtype)),
          c_int(n_rows), c_int(H), c_void_p(stream if stream is not None else current_stream_ptr()))


def qk_norm_rope_store(qkv: torch.Tensor, T: int, n_heads: int, n_kv: int, head_dim: int,
                       q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                       inv_freq: Optional[torch.Tensor], rotary: int, positions: torch.Tensor, seq_of: torch.Tensor,
                       block_table: torch.Tensor, page: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                       q_out: torch.Tensor, write_kv: bool = True, err: Optional[torch.Tensor] = None,
                       stream: Optional[int] = None) -> None:
    """Per head: optional RMSNorm, rotate-half rotation, q to ``q_out``, k/v into their pages."""
    _check(qkv, "qkv")
    _check(q_out, "q_out", qkv.dtype)
    _check(k_pool, "k_pool", qkv.dtype)
    _check(v_pool, "v_pool", qkv.dtype)
    _check(positions, "positions", torch.int32)
    _check(seq_of, "seq_of", torch.int32)
    _check(block_table, "block_table", torch.int32)
    for w, n in ((q_norm_w, "q_norm_w"), (k_norm_w, "k_norm_w"), (inv_freq, "inv_freq")):
        if w is not None:
            _check(w, n, torch.float32)
    if k_pool.dim() != 4 or k_pool.shape[1] != n_kv or k_pool.shape[2] != page or k_pool.shape[3] != head_dim:
        raise KernelError(f"qk_norm_rope_store: key pool {tuple(k_pool.shape)} is not [pages, {n_kv}, {page}, {head_dim}]")
    if v_pool.shape != k_pool.shape:
        raise KernelError("qk_norm_rope_store: key and value pools differ in shape")
    if inv_freq is not None and inv_freq.numel() * 2 != rotary:
        raise KernelError(f"qk_norm_rope_store: {inv_freq.numel()} frequencies for a rotation of {rotary}")
    lib = _lib("elementwise")
    _call(lib, lib.ember_qk_norm_rope_store, _p(qkv), c_int(dtype_code(qkv.dtype)), c_int(T), c_int(qkv.shape[-1]),
          c_int(n_heads), c_int(n_kv), c_int(head_dim), _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(inv_freq),
          c_int(rotary if inv_freq is not None else 0), _p(positions), _p(seq_of), _p(block_table),
          c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), _p(q_out), _p(k_pool), _p(v_pool),
          c_int(1 if write_kv else 0), _p(err), c_void_p(stream if stream is not None else current_stream_ptr()))


def qk_norm_rope_store_sums_usable(head_dim: int, rotary: int, width: int) -> bool:
    """Whether the head kernel can take a product's fp32 sums (heads of 128 rotated whole or not at all)."""
    return head_dim == 128 and rotary in (0, 128) and width % 8 == 0


def qk_norm_rope_store_sums(sums: torch.Tensor, T: int, n_heads: int, n_kv: int, q_norm_w: Optional[torch.Tensor],
                            k_norm_w: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor],
                            positions: torch.Tensor, seq_of: torch.Tensor, block_table: torch.Tensor, page: int,
                            k_pool: torch.Tensor, v_pool: torch.Tensor, q_out: torch.Tensor, write_kv: bool = True,
                            err: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """``qk_norm_rope_store`` on the fp32 sums [T, (n_heads + 2 n_kv) * 128] a product left in its scratch
    (``gemm_tc`` with ``EPI_SUMS``): queries and cache are bf16, and every sum read is set back to zero."""
    _check(sums, "sums", torch.float32)
    _check(q_out, "q_out", torch.bfloat16)
    _check(k_pool, "k_pool", torch.bfloat16)
    _check(v_pool, "v_pool", torch.bfloat16)
    _check(positions, "positions", torch.int32)
    _check(seq_of, "seq_of", torch.int32)
    _check(block_table, "block_table", torch.int32)
    for w, n in ((q_norm_w, "q_norm_w"), (k_norm_w, "k_norm_w"), (inv_freq, "inv_freq")):
        if w is not None:
            _check(w, n, torch.float32)
    if sums.dim() != 2 or sums.shape[0] < T or sums.shape[1] != (n_heads + 2 * n_kv) * 128:
        raise KernelError(f"qk_norm_rope_store_sums: sums {tuple(sums.shape)} for {T} tokens and {n_heads}/{n_kv} heads of 128")
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, 128) or v_pool.shape != k_pool.shape:
        raise KernelError(f"qk_norm_rope_store_sums: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, 128]")
    if inv_freq is not None and inv_freq.numel() != 64:
        raise KernelError(f"qk_norm_rope_store_sums: {inv_freq.numel()} frequencies for heads of 128")
    if q_out.numel() < T * n_heads * 128 or positions.numel() < T or seq_of.numel() < T:
        raise KernelError("qk_norm_rope_store_sums: query buffer or token arrays too small")
    lib = _lib("elementwise")
    _call(lib, lib.ember_qk_norm_rope_store_sums, _p(sums), c_int(T), c_int(sums.shape[1]), c_int(n_heads), c_int(n_kv),
          _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(inv_freq), c_int(128 if inv_freq is not None else 0), _p(positions),
          _p(seq_of), _p(block_table), c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), _p(q_out),
          _p(k_pool), _p(v_pool), c_int(1 if write_kv else 0), _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def wait_limit_probe(limit_ns: int, err: torch.Tensor, waited_ns: torch.Tensor, stream: Optional[int] = None) -> None:
    """Runs the kernels' bounded barrier wait on a barrier nobody arrives at, with a limit of ``limit_ns`` (at most
    100 ms): the wait gives up, the kernel returns, ``err`` gets the wait-limit bit and ``waited_ns`` (int64[1])
    how long the wait lasted.  For tests of the error path; nothing hangs."""
    _check(err, "err", torch.int32)
    _check(waited_ns, "waited_ns", torch.int64)
    lib = _lib("elementwise")
    _call(lib, lib.ember_wait_limit_probe, ctypes.c_ulonglong(int(limit_ns)), _p(err), _p(waited_ns),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def silu_mul_interleaved(x: torch.Tensor, out: torch.Tensor, n_out: int, stream: Optional[int] = None) -> None:
    _check(x, "x")
    _check(out, "out", x.dtype)
    lib = _lib("elementwise")
    _call(lib, lib.ember_silu_mul_interleaved, _p(x), _p(out), c_int(dtype_code(x.dtype)), c_longlong(n_out),
          c_void_p(stream if stream is not None else current_stream_ptr()))


# ------------------------------------------------------------------------------------ GEMM
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, M: int, epilogue: int = EPI_STORE,
              bias: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """out (+)= a[:M] @ w.T on the fp32 SIMT pipes (true 32-bit when both are float32)."""
    _check(a, "a")
    _check(w, "w")
    _check(out, "out")
    N, K = w.shape
    if a.shape[-1] != K:
        raise KernelError(f"gemm: activations of width {a.shape[-1]} against weights {tuple(w.shape)}")
    n_out = N // 2 if epilogue in GATED_EPILOGUES else N
    want = a.dtype if epilogue in (EPI_STORE,) + GATED_EPILOGUES else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm: epilogue {epilogue} writes {want}, the output is {out.dtype}")
    if out.shape[-1] != n_out or out.numel() < M * n_out or a.numel() < M * K:
        raise KernelError(f"gemm: output {tuple(out.shape)} / input {tuple(a.shape)} do not fit M={M} N={n_out}")
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelError(f"gemm: bias of {bias.numel()} for N={N}")
    lib = _lib("gemm_simt")
    _call(lib, lib.ember_gemm_simt, _p(a), c_int(dtype_code(a.dtype)), c_int(K), _p(w), c_int(dtype_code(w.dtype)),
          c_int(K), _p(bias), _p(out), c_int(n_out), c_int(M), c_int(N), c_int(K), c_int(epilogue),
          c_void_p(stream if stream is not None else current_stream_ptr()))


# ------------------------------------------------------------------------------- attention
ATTENTION_MAX_GROUP = 32     # query heads per key/value head the general attention kernel takes (its ATT_MAX_ROWS)


def attention_tile_queries(group: int) -> int:
    """How many query tokens one tile of the general attention kernel may hold."""
    lib = _lib("attention")
    n = lib.ember_attention_tile_queries(c_int(group))
    if n <= 0:
        raise KernelError(f"attention: {group} query heads per key/value head is more than the kernel takes")
    return n


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, T: int,
              n_heads: int, n_kv: int, head_dim: int, tiles: torch.Tensor, n_tiles: int, tile_q: int,
              block_table: torch.Tensor, page: int, window: int, scale: float, n_splits: int = 1,
              split_keys: int = 0, part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
              err: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """Causal attention of the step's tokens over the paged cache (general SIMT kernel)."""
    _check(q, "q")
    _check(out, "out", q.dtype)
    _check(k_pool, "k_pool", q.dtype)
    _check(v_pool, "v_pool", q.dtype)
    _check(tiles, "tiles", torch.int32)
    _check(block_table, "block_table", torch.int32)
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, {head_dim}]")
    if q.numel() < T * n_heads * head_dim or out.numel() < T * n_heads * head_dim:
        raise KernelError("attention: q/out too small for the step")
    if n_splits > 1 and (part_o is not None or part_ml is not None or n_splits > ATTENTION_CLUSTER_SPLITS):
        _check(part_o, "part_o", torch.float32)
        _check(part_ml, "part_ml", torch.float32)
        if part_o.numel() < T * n_heads * n_splits * head_dim or part_ml.numel() < T * n_heads * n_splits * 2:
            raise KernelError("attention: split buffers too small")
    lib = _lib("attention")
    _call(lib, lib.ember_attention, _p(q), _p(k_pool), _p(v_pool), _p(out), c_int(dtype_code(q.dtype)), c_int(T),
          c_int(n_heads), c_int(n_kv), c_int(head_dim), _p(tiles), c_int(n_tiles), c_int(tile_q), _p(block_table),
          c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), c_int(window), c_float(scale),
          c_int(n_splits), c_int(split_keys), _p(part_o), _p(part_ml), _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


# -------------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor, rows: int,
           stream: Optional[int] = None) -> None:
    """out[r] = token drawn from logits[r] under the packed 32-byte parameter row r."""
    _check(logits, "logits", torch.float32)
    _check(params, "params", torch.uint8)
    _check(out, "out", torch.int32)
    if logits.dim() != 2 or logits.shape[0] < rows or params.numel() < rows * 32 or out.numel() < rows:
        raise KernelError("sample: buffers do not fit the rows")
    lib = _lib("sampling")
    _call(lib, lib.ember_sample, _p(logits), c_int(rows), c_int(logits.shape[1]), _p(params), _p(out),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def argmax(logits: torch.Tensor, out: torch.Tensor, rows: int, part_v: torch.Tensor, part_i: torch.Tensor,
           stream: Optional[int] = None) -> None:
    """out[r] = index of the largest logit of row r, lowest index on ties (greedy sampling)."""
    _check(logits, "logits", torch.float32)
    _check(out, "out", torch.int32)
    _check(part_v, "part_v", torch.float32)
    _check(part_i, "part_i", torch.int32)
    if logits.dim() != 2 or logits.shape[0] < rows or out.numel() < rows or part_v.numel() < rows * 32 or part_i.numel() < rows * 32:
        raise KernelError("argmax: buffers do not fit the rows")
    lib = _lib("sampling")
    _call(lib, lib.ember_argmax, _p(logits), c_int(rows), c_int(logits.shape[1]), _p(part_v), _p(part_i), _p(out),
          c_void_p(stream if stream is not None else current_stream_ptr()))


# ------------------------------------------------------------- tensor-core kernels (bf16)
_tc_scratch = {}
_num_sms = {}
TC_ENABLED = True          # tests switch the tensor-core kernels off to check the general ones alone


def _sms(device) -> int:
    n = _num_sms.get(device)
    if n is None:
        n = torch.cuda.get_device_properties(device).multi_processor_count
        _num_sms[device] = n
    return n


_scratch_version = 0


def scratch_version() -> int:
    """Grows whenever the split-K scratch is (re)allocated: a captured CUDA graph holds the old address and must
    not be replayed afterwards."""
    return _scratch_version


def reserve_scratch(device, floats: int) -> torch.Tensor:
    """Makes the split-K scratch at least ``floats`` long.  A ``Linear`` reserves 128 x its output width when it
    is built, so that a loaded model never grows the scratch inside a step."""
    global _scratch_version
    device = torch.device(device)
    t = _tc_scratch.get(device)
    if t is None or t.numel() < floats:
        t = torch.zeros(max(int(floats), 1 << 20), dtype=torch.float32, device=device)
        _tc_scratch[device] = t
        _scratch_version += 1
    return t


def zero_scratch(device) -> None:
    t = _tc_scratch.get(torch.device(device))
    if t is not None:
        t.zero_()


def _scratch(device, floats: int) -> torch.Tensor:
    """Zero-filled fp32 scratch for split-K partial sums; the kernels leave it zeroed."""
    return reserve_scratch(device, floats)


def gemm_tc_usable(x: torch.Tensor, w: torch.Tensor, bias, epilogue: int) -> bool:
    """Whether the tcgen05 product takes these operands: bf16 activations and weights, no bias,
    K a multiple of 8 (TMA row pitch), an even N for the gated epilogue."""
    if not TC_ENABLED or bias is not None or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    n, k = w.shape
    return k % 8 == 0 and not (epilogue in GATED_EPILOGUES and n % 2)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, M: int, epilogue: int = EPI_STORE,
            err: Optional[torch.Tensor] = None, stream: Optional[int] = None, split_mode: int = 0) -> None:
    """out (+)= a[:M] @ w.T on the tcgen05 tensor cores (bf16 in, fp32 accumulate).  With ``EPI_SUMS`` (``out`` None,
    at most 128 tokens) the fp32 sums are left in the split-K scratch and returned as a view [M, N]: whoever reads
    them sets them back to zero (``qk_norm_rope_store_sums``).
    ``split_mode``: how split-K partial sums are combined (0 automatic, 1 atomics, 2 cluster); 3 runs
    prefill-sized products one tile per block instead of persistently, 4 on pairs of SMs whenever the device
    takes them, 5 never on pairs (for tests and tuning)."""
    _check(a, "a", torch.bfloat16)
    _check(w, "w", torch.bfloat16)
    N, K = w.shape
    if a.shape[-1] != K:
        raise KernelError(f"gemm: activations of width {a.shape[-1]} against weights {tuple(w.shape)}")
    if epilogue == EPI_SUMS:
        if out is not None or not 0 < M <= 128 or a.numel() < M * K:
            raise KernelError(f"gemm: the sums of M={M} tokens stay in the scratch only for 1..128 tokens and without an output")
        scratch = _scratch(a.device, M * N)
        lib = _lib("gemm_tc")
        _call(lib, lib.ember_gemm_tc, _p(a), _p(w), c_void_p(0), c_int(N), c_int(M), c_int(N), c_int(K), c_int(epilogue),
              _p(scratch), c_longlong(scratch.numel()), c_int(_sms(a.device)), c_int(split_mode), _p(err),
              c_void_p(stream if stream is not None else current_stream_ptr()))
        return scratch[:M * N].view(M, N)
    _check(out, "out")
    n_out = N // 2 if epilogue in GATED_EPILOGUES else N
    want = torch.bfloat16 if epilogue in (EPI_STORE,) + GATED_EPILOGUES else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm: epilogue {epilogue} writes {want}, the output is {out.dtype}")
    if out.shape[-1] != n_out or out.numel() < M * n_out or a.numel() < M * K:
        raise KernelError(f"gemm: output {tuple(out.shape)} / input {tuple(a.shape)} do not fit M={M} N={n_out}")
    scratch = _scratch(a.device, min(M, 128) * N) if M <= 128 else None
    lib = _lib("gemm_tc")
    _call(lib, lib.ember_gemm_tc, _p(a), _p(w), _p(out), c_int(n_out), c_int(M), c_int(N), c_int(K), c_int(epilogue),
          _p(scratch), c_longlong(scratch.numel() if scratch is not None else 0), c_int(_sms(a.device)), c_int(split_mode),
          _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def gemm_tc_qkv_usable(x: torch.Tensor, w: torch.Tensor, bias, M: int, n_heads: int, n_kv: int, head_dim: int,
                       rotary: int) -> bool:
    """Whether the fused projection takes this step: bf16, no bias, heads of 128 rotated whole (or not at all),
    more than 128 tokens or at most 16 (the rule of ember_gemm_tc_qkv_supported)."""
    if not gemm_tc_usable(x, w, bias, EPI_STORE):
        return False
    n, k = w.shape
    return (0 < M <= 16 or M > 128) and head_dim == 128 and rotary in (0, 128) and n == (n_heads + 2 * n_kv) * 128


# From how many tokens on a step's q/k/v product finishes the heads itself.  Measured at the 1.7B shape, product +
# head kernel against the fused product: 18.2 / 18.8 us at 256 tokens, 19.7 / 18.8 at 512, 38.2 / 29.3 at 2,048,
# 74.5 / 51.3 at 4,096 (below, the step is one or two tiles an SM and the longer epilogue has no next tile to
# hide behind).
QKV_FUSE_MIN_TOKENS = 512
# Up to how many tokens a decode step's q/k/v product does (product + head kernel against the fused product, in a
# graph: 8.4 / 6.2 us at 1 token, 9.1 / 7.6 at 8, 9.4 / 10.1 at 16: a block of the cluster finishes its share of
# the tokens one after the other, and only the first two are prepared while the product runs).
QKV_FUSE_MAX_DECODE_TOKENS = 8


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, T: int, out: torch.Tensor, stream: Optional[int] = None) -> None:
    """out[i // 2, t] = (cos_i, cos_{i+1}, sin_i, sin_{i+1}) of float(positions[t]) * inv_freq[i] in fp32;
    ``out`` is [frequencies / 2, tokens a row, 4] (token-minor: what the rotating epilogue reads)."""
    _check(positions, "positions", torch.int32)
    _check(inv_freq, "inv_freq", torch.float32)
    _check(out, "out", torch.float32)
    half = inv_freq.numel()
    if out.dim() != 3 or out.shape[0] != half // 2 or out.shape[2] != 4 or out.shape[1] < T or half % 2:
        raise KernelError(f"rope_table: output {tuple(out.shape)} for {half} frequencies and {T} tokens")
    lib = _lib("elementwise")
    _call(lib, lib.ember_rope_table, _p(positions), _p(inv_freq), c_int(T), c_int(half), c_int(out.shape[1]), _p(out),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def gemm_tc_qkv(a: torch.Tensor, w: torch.Tensor, M: int, n_heads: int, n_kv: int, q_norm_w: Optional[torch.Tensor],
                k_norm_w: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                inv_freq: Optional[torch.Tensor], positions: torch.Tensor,
                seq_of: torch.Tensor, block_table: torch.Tensor, page: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                q_out: torch.Tensor, write_kv: bool = True, err: Optional[torch.Tensor] = None,
                stream: Optional[int] = None, split_mode: int = 0) -> None:
    """[q | k | v] = a[:M] @ w.T on the tcgen05 tensor cores with the heads finished in the epilogue: RMSNorm and
    rotation of query and key heads in fp32 on the accumulator, queries to ``q_out``, keys and values into their
    cache pages.  More than 128 tokens rotate with ``cos_sin`` [32, tokens a row, 4] from ``rope_table``, at most
    16 with the frequencies ``inv_freq`` [64] (both None: no rotation).  Heads are 128 wide."""
    _check(a, "a", torch.bfloat16)
    _check(w, "w", torch.bfloat16)
    _check(q_out, "q_out", torch.bfloat16)
    _check(k_pool, "k_pool", torch.bfloat16)
    _check(v_pool, "v_pool", torch.bfloat16)
    _check(positions, "positions", torch.int32)
    _check(seq_of, "seq_of", torch.int32)
    _check(block_table, "block_table", torch.int32)
    for t, n in ((q_norm_w, "q_norm_w"), (k_norm_w, "k_norm_w"), (cos_sin, "cos_sin"), (inv_freq, "inv_freq")):
        if t is not None:
            _check(t, n, torch.float32)
    N, K = w.shape
    if a.shape[-1] != K or a.numel() < M * K:
        raise KernelError(f"gemm_qkv: activations {tuple(a.shape)} against weights {tuple(w.shape)} for M={M}")
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, 128) or v_pool.shape != k_pool.shape:
        raise KernelError(f"gemm_qkv: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, 128]")
    if q_out.numel() < M * n_heads * 128 or positions.numel() < M or seq_of.numel() < M:
        raise KernelError("gemm_qkv: query buffer or token arrays too small")
    if inv_freq is not None and inv_freq.numel() != 64:
        raise KernelError(f"gemm_qkv: {inv_freq.numel()} frequencies for heads of 128")
    if cos_sin is not None and (cos_sin.dim() != 3 or cos_sin.shape[0] != 32 or cos_sin.shape[1] < M or cos_sin.shape[2] != 4):
        raise KernelError(f"gemm_qkv: rotation table {tuple(cos_sin.shape)} is not [32, >= {M}, 4]")
    lib = _lib("gemm_tc")
    _call(lib, lib.ember_gemm_tc_qkv, _p(a), _p(w), c_int(M), c_int(N), c_int(K), c_int(n_heads), c_int(n_kv),
          _p(q_norm_w), _p(k_norm_w), c_float(eps), _p(cos_sin), c_int(cos_sin.shape[1] if cos_sin is not None else 0), _p(inv_freq), _p(positions), _p(seq_of), _p(block_table),
          c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), _p(q_out), _p(k_pool), _p(v_pool),
          c_int(1 if write_kv else 0), c_int(_sms(a.device)), c_int(split_mode), _p(err),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def num_sms(device) -> int:
    return _sms(device)


def attention_tc_supported(head_dim: int, group: int, page_tokens: int, mode: int) -> bool:
    """Whether the tensor-core attention takes this geometry (mode 0: prompt portions, 1: single tokens)."""
    # the same rule as ember_attention_tc_supported, stated here so that a model that cannot use the
    # kernels never loads (or compiles) their library
    if not TC_ENABLED or head_dim not in (64, 128) or page_tokens not in (16, 32, 64) or group < 1:
        return False
    return group <= 16 if mode == 1 else group <= 64


ATTENTION_CLUSTER_SPLITS = 8     # key splits of a decode tile that one thread-block cluster can merge


def attention_tc_tile_queries(group: int) -> int:
    return 64 // group if 1 <= group <= 64 else 0


FA_ENABLED = True


def attention_fa_supported(head_dim: int, group: int, page_tokens: int) -> bool:
    """Whether the tcgen05 prefill attention takes this geometry (the rule of ember_attention_fa_supported)."""
    return (TC_ENABLED and FA_ENABLED and head_dim == 128 and page_tokens in (16, 32, 64)
            and 1 <= group <= 128 and 128 % group == 0)


def attention_fa_tile_queries(group: int) -> int:
    return 128 // group


def attention_fa(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, n_heads: int,
                 n_kv: int, head_dim: int, tiles: torch.Tensor, n_tiles: int, block_table: torch.Tensor, page: int,
                 window: int, scale: float, err: Optional[torch.Tensor] = None, stream: Optional[int] = None,
                 softcap: float = 0.0, chunk: int = 0) -> None:
    """bf16 causal attention of prompt portions on tcgen05 tensor cores (S and O in tensor memory).  ``softcap`` > 0: the
    scaled score becomes softcap * tanh(score / softcap); ``chunk`` > 0: position i sees j only if
    floor(i / chunk) == floor(j / chunk)."""
    _check(q, "q", torch.bfloat16)
    _check(out, "out", torch.bfloat16)
    _check(k_pool, "k_pool", torch.bfloat16)
    _check(v_pool, "v_pool", torch.bfloat16)
    _check(tiles, "tiles", torch.int32)
    _check(block_table, "block_table", torch.int32)
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, {head_dim}]")
    lib = _lib("attention_fa")
    _call(lib, lib.ember_attention_fa, _p(q), _p(k_pool), _p(v_pool), _p(out), c_int(n_heads), c_int(n_kv), c_int(head_dim),
          _p(tiles), c_int(n_tiles), _p(block_table), c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]),
          c_int(window), c_float(scale), _p(err), c_float(softcap), c_int(chunk),
          c_void_p(stream if stream is not None else current_stream_ptr()))


def attention_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, mode: int,
                 n_heads: int, n_kv: int, head_dim: int, tiles: torch.Tensor, n_tiles: int, block_table: torch.Tensor,
                 page: int, window: int, scale: float, n_splits: int = 1, split_keys: int = 0,
                 part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                 err: Optional[torch.Tensor] = None, stream: Optional[int] = None, softcap: float = 0.0, chunk: int = 0) -> None:
    """bf16 attention over the paged cache on tensor cores (TMA-fed); ``softcap`` > 0 caps the scaled scores by a tanh,
    ``chunk`` > 0 lets position i see j only if floor(i / chunk) == floor(j / chunk).  ``mode`` 0 takes tiles of
    prompt portions, 1 takes single-token tiles and may split their key range: with ``part_o`` / ``part_ml`` the
    splits' partial results go through those buffers and a second kernel merges them; without them (at most 8
    splits) the splits of a tile are a thread-block cluster and are merged in shared memory."""
    _check(q, "q", torch.bfloat16)
    _check(out, "out", torch.bfloat16)
    _check(k_pool, "k_pool", torch.bfloat16)
    _check(v_pool, "v_pool", torch.bfloat16)
    _check(tiles, "tiles", torch.int32)
    _check(block_table, "block_table", torch.int32)
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (n_kv, page, head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention: pools {tuple(k_pool.shape)} are not [pages, {n_kv}, {page}, {head_dim}]")
    if n_splits > 1 and (part_o is not None or part_ml is not None or n_splits > ATTENTION_CLUSTER_SPLITS):
        _check(part_o, "part_o", torch.float32)
        _check(part_ml, "part_ml", torch.float32)
        if part_o.numel() < n_tiles * n_heads * n_splits * head_dim or part_ml.numel() < n_tiles * n_heads * n_splits * 2:
            raise KernelError("attention: split buffers too small")
    lib = _lib("attention_tc")
    _call(lib, lib.ember_attention_tc, _p(q), _p(k_pool), _p(v_pool), _p(out), c_int(mode), c_int(n_heads), c_int(n_kv),
          c_int(head_dim), _p(tiles), c_int(n_tiles), _p(block_table), c_int(block_table.shape[-1]), c_int(page),
          c_int(k_pool.shape[0]), c_int(window), c_float(scale), c_int(n_splits), c_int(split_keys), _p(part_o),
          _p(part_ml), _p(err), c_float(softcap), c_int(chunk), c_void_p(stream if stream is not None else current_stream_ptr()))


# ------------------------------------------------ norms and gates around a sublayer (csrc/norm_gate.cu)
def _stream(stream):
    return c_void_p(stream if stream is not None else current_stream_ptr())


def _off(t: torch.Tensor, elements: int = 0):
    """Address of element ``elements`` of a device tensor."""
    return c_void_p(t.data_ptr() + elements * t.element_size())


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, out: torch.Tensor,
               n_rows: int, rows: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """out[r] = (x - mean) / sqrt(var + eps) * weight + bias over x[rows[r] or r]; x fp32, statistics fp32."""
    _check(x, "x", torch.float32)
    _check(weight, "weight", torch.float32)
    _check(out, "out")
    H = x.shape[-1]
    if weight.numel() != H or out.shape[-1] != H or out.numel() < n_rows * H or (bias is not None and bias.numel() != H):
        raise KernelError(f"layer_norm: width {H}, weight {tuple(weight.shape)}, out {tuple(out.shape)} for {n_rows} rows")
    if rows is not None:
        _check(rows, "rows", torch.int32)
    lib = _lib("norm_gate")
    _call(lib, lib.ember_layer_norm, _p(x), _p(rows), _p(weight), _p(bias), c_float(eps), _p(out), c_int(dtype_code(out.dtype)),
          c_int(n_rows), c_int(H), _stream(stream))


def gated_norm_add(y: torch.Tensor, gate_logits: Optional[torch.Tensor], weight: torch.Tensor, bias: Optional[torch.Tensor],
                   eps: float, centred: bool, residual: torch.Tensor, n_rows: int, gate_bias: Optional[torch.Tensor] = None,
                   rounded: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """residual[r] += norm(y[r] * sigmoid(gate_logits[r] + gate_bias)): a layer norm (``centred``) or an RMS norm,
    all fp32.  ``rounded`` (bfloat16, the residual's shape) also receives the new rows, rounded once."""
    for t, n in ((y, "y"), (weight, "weight"), (residual, "residual")):
        _check(t, n, torch.float32)
    H = residual.shape[-1]
    if y.shape[-1] != H or weight.numel() != H or y.numel() < n_rows * H or residual.numel() < n_rows * H:
        raise KernelError(f"gated_norm_add: rows of {H}, y {tuple(y.shape)}, weight {tuple(weight.shape)}")
    if gate_logits is not None:
        _check(gate_logits, "gate_logits", torch.float32)
        if gate_logits.shape[-1] != H or gate_logits.numel() < n_rows * H:
            raise KernelError("gated_norm_add: the gate does not fit the rows")
    lib = _lib("norm_gate")
    if gate_bias is not None:
        _check(gate_bias, "gate_bias", torch.float32)
        if gate_bias.numel() != H:
            raise KernelError("gated_norm_add: the gate's bias does not fit the rows")
    if rounded is not None:
        _check(rounded, "rounded", torch.bfloat16)
        if rounded.shape[-1] != H or rounded.numel() < n_rows * H:
            raise KernelError("gated_norm_add: the rounded copy does not fit the rows")
    _call(lib, lib.ember_gated_norm_add, _p(y), _p(gate_logits), _p(gate_bias), _p(weight), _p(bias), c_float(eps), c_int(1 if centred else 0),
          _p(residual), _p(rounded), c_int(n_rows), c_int(H), _stream(stream))


def scaled_add_norm(y: torch.Tensor, y_bias: Optional[torch.Tensor], alpha: float, weight: torch.Tensor, bias: Optional[torch.Tensor],
                    eps: float, centred: bool, residual: torch.Tensor, n_rows: int, rounded: Optional[torch.Tensor] = None,
                    stream: Optional[int] = None) -> None:
    """residual[r] = norm(alpha * residual[r] + y[r] + y_bias) in place: the norm after the residual sum, a layer norm
    (``centred``) or an RMS norm, all fp32.  ``rounded`` (bfloat16) also receives the new rows, rounded once."""
    for t, n in ((y, "y"), (weight, "weight"), (residual, "residual")) + (((y_bias, "y_bias"),) if y_bias is not None else ()) + \
            (((bias, "bias"),) if bias is not None else ()):
        _check(t, n, torch.float32)
    H = residual.shape[-1]
    if y.shape[-1] != H or weight.numel() != H or y.numel() < n_rows * H or residual.numel() < n_rows * H or \
            (y_bias is not None and y_bias.numel() != H) or (bias is not None and bias.numel() != H):
        raise KernelError(f"scaled_add_norm: rows of {H}, y {tuple(y.shape)}, weight {tuple(weight.shape)}")
    if rounded is not None:
        _check(rounded, "rounded", torch.bfloat16)
        if rounded.shape[-1] != H or rounded.numel() < n_rows * H:
            raise KernelError("scaled_add_norm: the rounded copy does not fit the rows")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_scaled_add_norm, _p(y), _p(y_bias), c_float(alpha), _p(weight), _p(bias), c_float(eps), c_int(1 if centred else 0),
          _p(residual), _p(rounded), c_int(n_rows), c_int(H), _stream(stream))


def pair_norm_sum(a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, eps: float, out: torch.Tensor, n_rows: int,
                  accumulate: bool = False, stream: Optional[int] = None) -> None:
    """out[r] (+)= wa * a[r] / rms(a[r]) + wb * b[r] / rms(b[r]), each root mean square over the whole row (eps inside the
    root); all fp32."""
    for t, n in ((a, "a"), (wa, "wa"), (b, "b"), (wb, "wb"), (out, "out")):
        _check(t, n, torch.float32)
    H = out.shape[-1]
    if a.shape[-1] != H or b.shape[-1] != H or wa.numel() != H or wb.numel() != H or min(a.numel(), b.numel(), out.numel()) < n_rows * H:
        raise KernelError("pair_norm_sum: buffers do not fit the rows")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_pair_norm_sum, _p(a), _p(wa), _p(b), _p(wb), c_float(eps), _p(out), c_int(1 if accumulate else 0), c_int(n_rows),
          c_int(H), _stream(stream))


def add_row_bias(y: torch.Tensor, bias: torch.Tensor, n_rows: int, stream: Optional[int] = None) -> None:
    """y[r] += bias for the first ``n_rows`` rows (fp32)."""
    _check(y, "y", torch.float32)
    _check(bias, "bias", torch.float32)
    H = y.shape[-1]
    if bias.numel() != H or y.numel() < n_rows * H:
        raise KernelError("add_row_bias: buffers do not fit")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_add_row_bias, _p(y), _p(bias), c_int(n_rows), c_int(H), _stream(stream))


def round_rows(x: torch.Tensor, out: torch.Tensor, n: int, stream: Optional[int] = None) -> None:
    """out[:n] = bfloat16(x[:n]) (fp32 in): what a sublayer that reads the residual stream itself multiplies."""
    _check(x, "x", torch.float32)
    _check(out, "out", torch.bfloat16)
    if x.numel() < n or out.numel() < n:
        raise KernelError("round_rows: a buffer is too small")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_round_rows, _p(x), _p(out), c_longlong(n), _stream(stream))


GATE_NONE, GATE_SIGMOID_AFTER, GATE_SILU_BEFORE, GATE_SILU_AFTER = 0, 1, 2, 3


def group_norm_gate(x: torch.Tensor, x_col: int, gate: Optional[torch.Tensor], gate_col: int, weight: torch.Tensor,
                    per_group_weight: bool, eps: float, gate_mode: int, out: torch.Tensor, T: int, groups: int, width: int,
                    den: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """A token's ``groups * width`` values (fp32, from column ``x_col`` of x's rows), each group divided by its root
    mean square and multiplied by ``weight`` (one for all groups or one per group); the gate (fp32 rows, from column
    ``gate_col``) is a sigmoid or a silu after the norm, or a silu before it.  ``den`` (fp32 [T, groups, 4], what ``memory_scan``
    leaves): every group is first divided by max(|den[.., 3]|, den[.., 2]) + 1e-6."""
    _check(x, "x", torch.float32)
    _check(weight, "weight", torch.float32)
    _check(out, "out")
    if x.dim() != 2 or x.shape[0] < T or x_col + groups * width > x.shape[1] or out.numel() < T * groups * width:
        raise KernelError(f"group_norm_gate: {groups} groups of {width} from column {x_col} of {tuple(x.shape)}")
    if weight.numel() != (groups * width if per_group_weight else width):
        raise KernelError(f"group_norm_gate: weight of {weight.numel()} for {groups} groups of {width}")
    if gate_mode != GATE_NONE:
        _check(gate, "gate", torch.float32)
        if gate.dim() != 2 or gate.shape[0] < T or gate_col + groups * width > gate.shape[1]:
            raise KernelError("group_norm_gate: the gate does not fit")
    if den is not None:
        _check(den, "den", torch.float32)
        if den.numel() < T * groups * 4:
            raise KernelError("group_norm_gate: the denominators do not fit")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_group_norm_gate, _off(x, x_col), c_int(x.shape[1]), _off(gate, gate_col) if gate_mode else c_void_p(0),
          c_int(gate.shape[1] if gate_mode else 0), _p(weight), c_int(width if per_group_weight else 0), c_float(eps),
          c_int(gate_mode), _p(den), _p(out), c_int(dtype_code(out.dtype)), c_int(T), c_int(groups), c_int(width), _stream(stream))


def scaled_sum(x: torch.Tensor, a: float, y: Optional[torch.Tensor], b: float, out: torch.Tensor, n: int,
               accumulate: bool = False, stream: Optional[int] = None) -> None:
    """out[:n] (+)= a * x[:n] + b * y[:n], fp32."""
    for t, name in ((x, "x"), (out, "out")) + (((y, "y"),) if y is not None else ()):
        _check(t, name, torch.float32)
        if t.numel() < n:
            raise KernelError("scaled_sum: a buffer is too small")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_scaled_sum, _p(x), c_float(a), _p(y), c_float(b), _p(out), c_int(1 if accumulate else 0), c_longlong(n),
          _stream(stream))


def dynamic_tanh(x: torch.Tensor, alpha: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                 n_rows: int, rows: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """out[r] = tanh(alpha * x[rows[r] or r]) * weight + bias, element by element; x fp32, ``alpha`` a device scalar."""
    for t, n in ((x, "x"), (alpha, "alpha"), (weight, "weight")) + (((bias, "bias"),) if bias is not None else ()):
        _check(t, n, torch.float32)
    _check(out, "out")
    H = x.shape[-1]
    if weight.numel() != H or alpha.numel() != 1 or out.shape[-1] != H or out.numel() < n_rows * H or (bias is not None and bias.numel() != H):
        raise KernelError(f"dynamic_tanh: width {H}, weight {tuple(weight.shape)}, out {tuple(out.shape)} for {n_rows} rows")
    if rows is not None:
        _check(rows, "rows", torch.int32)
    lib = _lib("norm_gate")
    _call(lib, lib.ember_dynamic_tanh, _p(x), _p(rows), _p(alpha), _p(weight), _p(bias), _p(out), c_int(dtype_code(out.dtype)),
          c_int(n_rows), c_int(H), _stream(stream))


STREAMS_MAX = 16                 # copies of the residual stream the stream kernels take (their MAX_STREAMS)


def stream_read(X: torch.Tensor, streams: int, in_w: Optional[torch.Tensor], out: torch.Tensor, T: int,
                norm=None, stream: Optional[int] = None) -> None:
    """out[t] = sum_s in_w[s] * X[t, s] over the ``streams`` copies of the residual stream (X fp32 [T, streams width];
    ``in_w`` None: ones).  ``norm`` = (alpha, weight, bias): the sum goes through tanh(alpha u) * weight + bias."""
    _check(X, "X", torch.float32)
    _check(out, "out")
    H = out.shape[-1]
    if X.shape[-1] != streams * H or X.numel() < T * streams * H or out.numel() < T * H:
        raise KernelError(f"stream_read: {streams} copies of width {H} in rows of {X.shape[-1]}")
    if in_w is not None:
        _check(in_w, "in_w", torch.float32)
        if in_w.numel() != streams:
            raise KernelError("stream_read: one weight per copy")
    alpha, w, b = norm if norm is not None else (None, None, None)
    for t, n in ((alpha, "alpha"), (w, "weight"), (b, "bias")):
        if t is not None:
            _check(t, n, torch.float32)
    if norm is None and out.dtype != torch.float32:
        raise KernelError("stream_read: the plain sum is fp32")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_stream_read, _p(X), c_int(streams), _p(in_w), _p(alpha), _p(w), _p(b), _p(out), c_int(dtype_code(out.dtype)),
          c_int(T), c_int(H), _stream(stream))


def stream_write(X: torch.Tensor, streams: int, mix: Optional[torch.Tensor], out_w: Optional[torch.Tensor],
                 scale: Optional[torch.Tensor], multiplier: float, y: torch.Tensor, T: int, stream: Optional[int] = None) -> None:
    """Every copy r at once from the old copies: X[t, r] <- sum_s mix[s, r] X[t, s] + multiplier * out_w[r] * scale * y[t]
    (``mix`` fp32 [streams, streams] or None: the identity; ``out_w`` None: ones; ``scale`` fp32 [width] or None)."""
    _check(X, "X", torch.float32)
    _check(y, "y", torch.float32)
    H = y.shape[-1]
    if X.shape[-1] != streams * H or X.numel() < T * streams * H or y.numel() < T * H:
        raise KernelError(f"stream_write: {streams} copies of width {H} in rows of {X.shape[-1]}")
    for t, n, size in ((mix, "mix", streams * streams), (out_w, "out_w", streams), (scale, "scale", H)):
        if t is not None:
            _check(t, n, torch.float32)
            if t.numel() != size:
                raise KernelError(f"stream_write: {n} has {t.numel()} elements, not {size}")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_stream_write, _p(X), c_int(streams), _p(mix), _p(out_w), _p(scale), c_float(multiplier), _p(y), c_int(T),
          c_int(H), _stream(stream))


def stream_spread(x: torch.Tensor, X: torch.Tensor, streams: int, T: int, stream: Optional[int] = None) -> None:
    """X[t, s] = x[t] for every copy s (fp32)."""
    _check(x, "x", torch.float32)
    _check(X, "X", torch.float32)
    H = x.shape[-1]
    if X.shape[-1] != streams * H or X.numel() < T * streams * H or x.numel() < T * H:
        raise KernelError("stream_spread: buffers do not fit")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_stream_spread, _p(x), _p(X), c_int(streams), c_int(T), c_int(H), _stream(stream))


def stream_sum(X: torch.Tensor, streams: int, out: torch.Tensor, n_rows: int, rows: Optional[torch.Tensor] = None,
               stream: Optional[int] = None) -> None:
    """out[r] = sum over the copies of X[rows[r] or r] (fp32)."""
    _check(X, "X", torch.float32)
    _check(out, "out", torch.float32)
    H = out.shape[-1]
    if X.shape[-1] != streams * H or out.numel() < n_rows * H:
        raise KernelError("stream_sum: buffers do not fit")
    if rows is not None:
        _check(rows, "rows", torch.int32)
    lib = _lib("norm_gate")
    _call(lib, lib.ember_stream_sum, _p(X), _p(rows), c_int(streams), _p(out), c_int(n_rows), c_int(H), _stream(stream))


def logit_finish(logits: torch.Tensor, n: int, scale: float, cap: float, stream: Optional[int] = None) -> None:
    """logits[:n] <- cap * tanh(scale * logits / cap) in place (cap 0: scale * logits); fp32."""
    _check(logits, "logits", torch.float32)
    if logits.numel() < n:
        raise KernelError("logit_finish: the buffer is too small")
    lib = _lib("norm_gate")
    _call(lib, lib.ember_logit_finish, _p(logits), c_float(scale), c_float(cap), c_longlong(n), _stream(stream))


ACTIVATIONS = tuple(GATED_EPILOGUE_OF)      # what the gated epilogue of the products takes


# -------------------------------------------------------------------- recurrent mixers (csrc/recurrent.cu)
def _check_runs(query_start: torch.Tensor, slots: torch.Tensor, S: int) -> None:
    _check(query_start, "query_start", torch.int32)
    _check(slots, "slots", torch.int32)
    if query_start.numel() < S + 1 or slots.numel() < S:
        raise KernelError("the run arrays are shorter than the step")


def conv_silu(x: torch.Tensor, col: int, taps: torch.Tensor, bias: Optional[torch.Tensor], carry: torch.Tensor,
              carry_col: int, seq_of: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
              T: int, S: int, stream: Optional[int] = None, silu: bool = True) -> None:
    """Short causal convolution per channel + silu (``silu`` False: the convolution alone) over the step's runs.  ``x`` fp32 [T, ld]: channels are its
    columns col .. col + C; ``taps`` fp32 [C, n] (the last column meets the current token); ``carry`` fp32
    [slots, row]: a request's last n - 1 inputs live at columns carry_col .. carry_col + (n - 1) C of its row and
    are replaced by this step's."""
    for t, n in ((x, "x"), (taps, "taps"), (carry, "carry"), (out, "out")):
        _check(t, n, torch.float32)
    _check(seq_of, "seq_of", torch.int32)
    _check_runs(query_start, slots, S)
    C, n = taps.shape
    if x.dim() != 2 or x.shape[0] < T or col + C > x.shape[1] or out.numel() < T * C or carry.dim() != 2 or \
            carry_col + (n - 1) * C > carry.shape[1] or (bias is not None and bias.numel() != C):
        raise KernelError(f"conv_silu: {C} channels x {n} taps from column {col} of {tuple(x.shape)}, carry {tuple(carry.shape)}")
    lib = _lib("recurrent")
    _call(lib, lib.ember_conv_silu, _p(x), c_int(x.shape[1]), c_int(col), _p(taps), _p(bias), c_int(n), _off(carry, carry_col),
          c_longlong(carry.shape[1]), _p(seq_of), _p(query_start), _p(slots), _p(out), c_int(T), c_int(S), c_int(C),
          c_int(1 if silu else 0), _stream(stream))


def delta_scan(conv: torch.Tensor, beta: torch.Tensor, beta_col: int, a: torch.Tensor, a_col: int, dt_bias: torch.Tensor,
               A_log: torch.Tensor, state: torch.Tensor, out: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor,
               T: int, S: int, heads: int, kv_heads: int, dim: int, vdim: int, key_eps: float, stream: Optional[int] = None,
               per_head_decay: bool = False) -> None:
    """Delta rule with a decay per head and key channel over the step's runs; the state [slots, >= heads dim vdim]
    fp32 is read and left updated (``T`` tokens in ``S`` runs; T == S, a decode step, takes small blocks).  ``conv`` fp32 [T, q | k | v] after convolution and silu, ``beta`` logits at
    column beta_col, decay logits at column a_col of ``a``; out fp32 [T, heads vdim].  ``per_head_decay``: one decay
    logit (and one ``dt_bias``) per head instead of per head and key channel."""
    for t, n in ((conv, "conv"), (beta, "beta"), (a, "a"), (dt_bias, "dt_bias"), (A_log, "A_log"), (state, "state"), (out, "out")):
        _check(t, n, torch.float32)
    _check_runs(query_start, slots, S)
    if conv.shape[1] != 2 * kv_heads * dim + heads * vdim or beta_col + heads > beta.shape[1] or \
            a_col + heads * (1 if per_head_decay else dim) > a.shape[1] or \
            dt_bias.numel() != heads * (1 if per_head_decay else dim) or A_log.numel() != heads or \
            state.dim() != 2 or state.shape[1] < heads * dim * vdim:
        raise KernelError("delta_scan: buffers do not fit the head geometry")
    lib = _lib("recurrent")
    _call(lib, lib.ember_delta_scan, _p(conv), c_int(conv.shape[1]), _off(beta, beta_col), c_int(beta.shape[1]), _off(a, a_col),
          c_int(a.shape[1]), _p(dt_bias), _p(A_log), _p(state), c_longlong(state.shape[1]), _p(out), _p(query_start), _p(slots),
          c_int(T), c_int(S), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_float(key_eps),
          c_int(1 if per_head_decay else 0), _stream(stream))


def memory_scan(proj: torch.Tensor, off_q: int, off_k: int, off_v: int, off_i: int, off_f: int, bias_i: torch.Tensor,
                bias_f: torch.Tensor, cap: float, state: torch.Tensor, gates: torch.Tensor, out: torch.Tensor,
                query_start: torch.Tensor, slots: torch.Tensor, T: int, S: int, heads: int, dim: int, vdim: int,
                stream: Optional[int] = None) -> None:
    """Matrix memory with exponential input gate and running maximum over the step's runs.  ``proj`` fp32 [T, ld]
    holds q, k, v and the two gates' logits at the given columns; the state row of a request is S [heads, dim, vdim],
    n [heads, dim], m [heads].  Leaves out fp32 [T, heads vdim] = S^T q and ``gates`` fp32 [T, heads, 4] = (keep, put,
    e^-m, n . q): the read-out is out / (max(|n . q|, e^-m) + 1e-6), which ``group_norm_gate`` applies (``den``)."""
    for t, n in ((proj, "proj"), (bias_i, "bias_i"), (bias_f, "bias_f"), (state, "state"), (gates, "gates"), (out, "out")):
        _check(t, n, torch.float32)
    _check_runs(query_start, slots, S)
    if state.dim() != 2 or state.shape[1] < heads * dim * vdim + heads * dim + heads or bias_i.numel() != heads or \
            bias_f.numel() != heads or gates.numel() < proj.shape[0] * heads * 4:
        raise KernelError("memory_scan: buffers do not fit the head geometry")
    lib = _lib("recurrent")
    _call(lib, lib.ember_memory_scan, _p(proj), c_int(proj.shape[1]), c_int(off_q), c_int(off_k), c_int(off_v), c_int(off_i),
          c_int(off_f), _p(bias_i), _p(bias_f), c_float(cap), _p(state), c_longlong(state.shape[1]), _p(gates), _p(out),
          _p(query_start), _p(slots), c_int(T), c_int(S), c_int(heads), c_int(dim), c_int(vdim), _stream(stream))


def ssm_scan(conv: torch.Tensor, dt: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, A_log: torch.Tensor, skip: torch.Tensor,
             state: torch.Tensor, out: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor, T: int, S: int, heads: int,
             groups: int, n_state: int, vdim: int, stream: Optional[int] = None) -> None:
    """Selective state space with a scalar decay per head over the step's runs.  ``conv`` fp32 [T, x | B | C] after
    convolution and silu, raw step sizes at column dt_col of ``dt``; state [slots, >= heads n_state vdim] fp32."""
    for t, n in ((conv, "conv"), (dt, "dt"), (dt_bias, "dt_bias"), (A_log, "A_log"), (skip, "skip"), (state, "state"), (out, "out")):
        _check(t, n, torch.float32)
    _check_runs(query_start, slots, S)
    if conv.shape[1] != heads * vdim + 2 * groups * n_state or dt_col + heads > dt.shape[1] or \
            state.dim() != 2 or state.shape[1] < heads * n_state * vdim:
        raise KernelError("ssm_scan: buffers do not fit the head geometry")
    lib = _lib("recurrent")
    _call(lib, lib.ember_ssm_scan, _p(conv), c_int(conv.shape[1]), _off(dt, dt_col), c_int(dt.shape[1]), _p(dt_bias), _p(A_log),
          _p(skip), _p(state), c_longlong(state.shape[1]), _p(out), _p(query_start), _p(slots), c_int(T), c_int(S), c_int(heads),
          c_int(groups), c_int(n_state), c_int(vdim), _stream(stream))


def token_shift(x: torch.Tensor, mu: torch.Tensor, carry: torch.Tensor, carry_col: int, seq_of: torch.Tensor,
                query_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, T: int, S: int,
                stream: Optional[int] = None) -> None:
    """out[m, t] = x[t] + (x'[t] - x[t]) * mu[m] for every blend m (``mu`` fp32 [blends, width]), x' the row of the token
    before t in its request: the row above inside a run, else the request's carried row (columns carry_col .. + width of
    its row of ``carry`` fp32 [slots, row]; zeros for a new request).  The carried rows are then replaced by the runs'
    last rows.  ``out`` [blends, rows, width] has x's dtype."""
    _check(x, "x")
    _check(out, "out", x.dtype)
    _check(mu, "mu", torch.float32)
    _check(carry, "carry", torch.float32)
    _check(seq_of, "seq_of", torch.int32)
    _check_runs(query_start, slots, S)
    n_mix, C = mu.shape
    if x.shape[-1] != C or x.numel() < T * C or out.dim() != 3 or out.shape[0] != n_mix or out.shape[2] != C or out.shape[1] < T or \
            carry.dim() != 2 or carry_col + C > carry.shape[1]:
        raise KernelError(f"token_shift: {n_mix} blends of width {C}: x {tuple(x.shape)}, out {tuple(out.shape)}, carry {tuple(carry.shape)}")
    lib = _lib("recurrent")
    _call(lib, lib.ember_token_shift, _p(x), c_int(dtype_code(x.dtype)), _p(mu), c_int(n_mix), _off(carry, carry_col),
          c_longlong(carry.shape[1]), _p(seq_of), _p(query_start), _p(slots), _p(out), c_int(dtype_code(out.dtype)),
          c_longlong(out.shape[1] * C), c_int(T), c_int(S), c_int(C), _stream(stream))


def wkv_scan(proj: torch.Tensor, ld: int, off_r: int, off_k: int, off_v: int, z: torch.Tensor, z_col: int, w0: torch.Tensor,
             bonus: torch.Tensor, state: torch.Tensor, out: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor,
             T: int, S: int, heads: int, dim: int, vdim: int, stream: Optional[int] = None) -> None:
    """Time mixing over the step's runs: per head o = (S + diag(u) k v^T)^T r, then S <- diag(w) S + k v^T with
    w = exp(-exp(z + w0)) per key channel.  ``proj`` fp32 holds r, k, v in rows of ``ld`` elements starting ``off_*``
    elements behind its first (they may be separate blocks of one buffer); ``z`` fp32 rows hold the decay logits
    [heads dim] from column z_col; ``w0``, ``bonus`` fp32 [heads dim]; the state [slots, >= heads dim vdim] fp32 is read
    and left updated; out fp32 [T, heads vdim]."""
    for t, n in ((proj, "proj"), (z, "z"), (w0, "w0"), (bonus, "bonus"), (state, "state"), (out, "out")):
        _check(t, n, torch.float32)
    _check_runs(query_start, slots, S)
    last = (T - 1) * ld
    if max(off_r, off_k) + last + heads * dim > proj.numel() or off_v + last + heads * vdim > proj.numel() or \
            z_col + heads * dim > z.shape[1] or state.dim() != 2 or state.shape[1] < heads * dim * vdim or \
            out.numel() < T * heads * vdim or w0.numel() != heads * dim or bonus.numel() != heads * dim:
        raise KernelError("wkv_scan: buffers do not fit the head geometry")
    lib = _lib("recurrent")
    _call(lib, lib.ember_wkv_scan, _p(proj), c_int(ld), c_longlong(off_r), c_longlong(off_k), c_longlong(off_v), _off(z, z_col),
          c_int(z.shape[1]), _p(w0), _p(bonus), _p(state), c_longlong(state.shape[1]), _p(out), _p(query_start), _p(slots), c_int(T),
          c_int(S), c_int(heads), c_int(dim), c_int(vdim), _stream(stream))


# ------------------------------------------------------- attention without softmax (csrc/sigmoid_attention.cu)
def sigmoid_attention_tile_queries(group: int) -> int:
    """Query tokens per tile: a block's 16 rows are (token, head) pairs over the largest divisor of the group that
    is at most 16 (the rule of ember_sigmoid_attention_tile_queries)."""
    h = min(group, 16)
    while group % h:
        h -= 1
    return 16 // h


def rotate_store(qkv: torch.Tensor, T: int, heads: int, kv_heads: int, dim: int, vdim: int, inv_freq: Optional[torch.Tensor],
                 rotary: int, positions: torch.Tensor, seq_of: torch.Tensor, block_table: torch.Tensor, page: int,
                 k_pool: torch.Tensor, v_pool: torch.Tensor, q_out: torch.Tensor, write_kv: bool = True,
                 err: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """Rotation of query and key heads (first ``rotary`` elements, rotate-half pairs), queries to ``q_out``, keys
    [.., dim] and values [.., vdim] into their pages.  ``qkv`` is fp32 [T, q | k | v]."""
    _check(qkv, "qkv", torch.float32)
    _check(q_out, "q_out")
    _check(k_pool, "k_pool", q_out.dtype)
    _check(v_pool, "v_pool", q_out.dtype)
    for t, n in ((positions, "positions"), (seq_of, "seq_of"), (block_table, "block_table")):
        _check(t, n, torch.int32)
    if tuple(k_pool.shape[1:]) != (kv_heads, page, dim) or tuple(v_pool.shape[1:]) != (kv_heads, page, vdim) or \
            k_pool.shape[0] != v_pool.shape[0]:
        raise KernelError(f"rotate_store: pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit")
    if inv_freq is not None:
        _check(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() * 2 != rotary:
            raise KernelError(f"rotate_store: {inv_freq.numel()} frequencies for a rotation of {rotary}")
    if q_out.numel() < T * heads * dim or qkv.shape[0] < T:
        raise KernelError("rotate_store: buffers too small for the step")
    lib = _lib("sigmoid_attention")
    _call(lib, lib.ember_rotate_store, _p(qkv), c_int(qkv.shape[1]), c_int(T), c_int(heads), c_int(kv_heads), c_int(dim),
          c_int(vdim), _p(inv_freq), c_int(rotary if inv_freq is not None else 0), _p(positions), _p(seq_of), _p(block_table),
          c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), _p(q_out), _p(k_pool), _p(v_pool),
          c_int(dtype_code(q_out.dtype)), c_int(1 if write_kv else 0), _p(err), _stream(stream))


def sigmoid_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor, heads: int,
                      kv_heads: int, dim: int, vdim: int, tiles: torch.Tensor, n_tiles: int, block_table: torch.Tensor,
                      page: int, scale: float, head_bias: Optional[torch.Tensor], err: Optional[torch.Tensor] = None,
                      stream: Optional[int] = None) -> None:
    """out[t, h] = sum over keys j <= t of sigmoid(scale * q . k_j + head_bias[h]) * v_j (no normalisation)."""
    _check(q, "q")
    for t, n in ((out, "out"), (k_pool, "k_pool"), (v_pool, "v_pool")):
        _check(t, n, q.dtype)
    _check(tiles, "tiles", torch.int32)
    _check(block_table, "block_table", torch.int32)
    if head_bias is not None:
        _check(head_bias, "head_bias", torch.float32)
    if tuple(k_pool.shape[1:]) != (kv_heads, page, dim) or tuple(v_pool.shape[1:]) != (kv_heads, page, vdim):
        raise KernelError(f"sigmoid_attention: pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit")
    lib = _lib("sigmoid_attention")
    _call(lib, lib.ember_sigmoid_attention, _p(q), _p(k_pool), _p(v_pool), _p(out), c_int(dtype_code(q.dtype)), c_int(heads),
          c_int(kv_heads), c_int(dim), c_int(vdim), _p(tiles), c_int(n_tiles), _p(block_table), c_int(block_table.shape[-1]),
          c_int(page), c_int(k_pool.shape[0]), c_float(scale), _p(head_bias), _p(err), _stream(stream))


def gla_scan(proj: torch.Tensor, off_q: int, off_k: int, off_v: int, z: torch.Tensor, z_col: int, z_bias: Optional[torch.Tensor],
             decay_power: float, state: torch.Tensor, out: torch.Tensor, query_start: torch.Tensor, slots: torch.Tensor,
             T: int, S: int, heads: int, dim: int, vdim: int, stream: Optional[int] = None) -> None:
    """Gated linear attention over the step's runs: S <- diag(alpha) S + k v^T, o = S^T q per head, with
    alpha = sigmoid(z + z_bias)^decay_power per key channel and q times dim^-1/2.  ``proj`` fp32 [T, ld] holds q, k, v at
    the given columns, ``z`` fp32 rows hold the decay logits [heads dim] from column z_col; the state
    [slots, >= heads dim vdim] fp32 is read and left updated; out fp32 [T, heads vdim]."""
    for t, n in ((proj, "proj"), (z, "z"), (state, "state"), (out, "out")) + (((z_bias, "z_bias"),) if z_bias is not None else ()):
        _check(t, n, torch.float32)
    _check_runs(query_start, slots, S)
    ld = proj.shape[1]
    if max(off_q, off_k) + heads * dim > ld or off_v + heads * vdim > ld or z_col + heads * dim > z.shape[1] or \
            state.dim() != 2 or state.shape[1] < heads * dim * vdim or out.numel() < T * heads * vdim or \
            (z_bias is not None and z_bias.numel() != heads * dim):
        raise KernelError("gla_scan: buffers do not fit the head geometry")
    lib = _lib("recurrent")
    _call(lib, lib.ember_gla_scan, _p(proj), c_int(ld), c_int(off_q), c_int(off_k), c_int(off_v), _off(z, z_col), c_int(z.shape[1]),
          _p(z_bias), c_float(decay_power), _p(state), c_longlong(state.shape[1]), _p(out), _p(query_start), _p(slots), c_int(T),
          c_int(S), c_int(heads), c_int(dim), c_int(vdim), _stream(stream))


# ------------------------------------- softmax attention with a sink, whole-projection norms, latents (csrc/sink_attention.cu)
SINK_ATTENTION_ROWS = 32         # (query, head) rows of a tile of the kernel (its SA_MAX_ROWS)


def sink_attention_tile_queries(group: int) -> int:
    """Query tokens per tile: a block takes up to 32 (token, head) rows over up to 32 of the query heads of a key head."""
    return max(1, SINK_ATTENTION_ROWS // max(1, min(group, SINK_ATTENTION_ROWS)))


def _check_pages(k_pool, v_pool, kv_heads, page, dim, vdim, what):
    if k_pool.dim() != 4 or tuple(k_pool.shape[1:]) != (kv_heads, page, dim) or \
            (v_pool is not None and (tuple(v_pool.shape[1:]) != (kv_heads, page, vdim) or v_pool.shape[0] != k_pool.shape[0])):
        raise KernelError(f"{what}: pools {tuple(k_pool.shape)} / {tuple(v_pool.shape) if v_pool is not None else None} do not fit "
                          f"[pages, {kv_heads}, {page}, {dim} | {vdim}]")


def _check_head_gate(head_gate, T: int, heads: int, col: int = 0) -> None:
    if head_gate is not None:
        _check(head_gate, "head_gate", torch.float32)
        if head_gate.dim() != 2 or head_gate.shape[0] < T or col < 0 or head_gate.shape[1] < col + heads:
            raise KernelError(f"attention: a head gate of {tuple(head_gate.shape)} from column {col} for {T} tokens of {heads} heads")


def head_gate_apply(x: torch.Tensor, gate: torch.Tensor, gate_col: int, T: int, heads: int, vdim: int, stream: Optional[int] = None) -> None:
    """x[t, h, :] *= sigmoid(gate[t, gate_col + h]) in place (x [T, heads vdim] bfloat16 or float32, gate fp32 logits)."""
    _check(x, "x")
    _check_head_gate(gate, T, heads, gate_col)
    if gate is None or x.numel() < T * heads * vdim:
        raise KernelError("head_gate_apply: buffers do not fit the step")
    lib = _lib("sink_attention")
    _call(lib, lib.ember_head_gate_apply, _p(x), c_int(dtype_code(x.dtype)), _off(gate, gate_col), c_int(gate.shape[-1]), c_int(T),
          c_int(heads), c_int(vdim), _stream(stream))


def head_prepare_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], norm_mode: str, q_w: Optional[torch.Tensor],
                       k_w: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rotary: int, q_temp_coef: float,
                       q_temp_every: int, T: int, heads: int, kv_heads: int, dim: int, vdim: int, positions: torch.Tensor,
                       seq_of: torch.Tensor, block_table: torch.Tensor, page: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                       q_out: torch.Tensor, write_kv: bool = True, err: Optional[torch.Tensor] = None,
                       stream: Optional[int] = None) -> None:
    """A token's q/k/v (``qkv`` fp32 [T, q | k | v], plus ``bias``) made ready for attention: an RMS norm of queries and
    keys (``norm_mode`` "none", "whole": over the whole projection with weights of that size, "head": per head with
    weights of ``dim`` shared by the heads), the rotation of the first ``rotary`` elements of every query and key head
    (element i with i + rotary / 2, angle position * inv_freq[i]), the query times
    1 + q_temp_coef * ln(floor((position + 1) / q_temp_every) + 1) (``q_temp_every`` 0: not); queries to ``q_out``, keys and
    values into the token's page."""
    _check(qkv, "qkv", torch.float32)
    modes = {"none": 0, "whole": 1, "head": 2}
    if norm_mode not in modes:
        raise KernelError(f"head_prepare_store: norm mode {norm_mode!r}")
    qn, kn = heads * dim, kv_heads * dim
    for t, n, size in ((bias, "bias", qn + kn + kv_heads * vdim), (q_w, "q_w", qn if norm_mode == "whole" else dim),
                       (k_w, "k_w", kn if norm_mode == "whole" else dim), (inv_freq, "inv_freq", rotary // 2)):
        if t is not None:
            _check(t, n, torch.float32)
            if t.numel() != size:
                raise KernelError(f"head_prepare_store: {n} has {t.numel()} elements, not {size}")
    if norm_mode != "none" and (q_w is None or k_w is None):
        raise KernelError("head_prepare_store: a norm needs its weights")
    if rotary and inv_freq is None:
        raise KernelError("head_prepare_store: a rotation needs its frequencies")
    _check(positions, "positions", torch.int32)
    _check(seq_of, "seq_of", torch.int32)
    _check(block_table, "block_table", torch.int32)
    _check(q_out, "q_out")
    _check(k_pool, "k_pool", q_out.dtype)
    _check(v_pool, "v_pool", q_out.dtype)
    _check_pages(k_pool, v_pool, kv_heads, page, dim, vdim, "head_prepare_store")
    if qkv.dim() != 2 or qkv.shape[0] < T or qkv.shape[1] < qn + kn + kv_heads * vdim or q_out.numel() < T * qn:
        raise KernelError("head_prepare_store: buffers do not fit the step")
    lib = _lib("sink_attention")
    _call(lib, lib.ember_head_prepare_store, _p(qkv), c_int(qkv.shape[1]), _p(bias), c_int(modes[norm_mode]), _p(q_w), _p(k_w),
          c_float(eps), _p(inv_freq), c_int(rotary), c_float(q_temp_coef), c_int(q_temp_every), c_int(T), c_int(heads), c_int(kv_heads),
          c_int(dim), c_int(vdim), _p(positions), _p(seq_of), _p(block_table), c_int(block_table.shape[-1]), c_int(page),
          c_int(k_pool.shape[0]), _p(q_out), _p(k_pool), _p(v_pool), c_int(dtype_code(q_out.dtype)), c_int(1 if write_kv else 0),
          _p(err), _stream(stream))


def whole_norm_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                     eps: float, T: int, heads: int, kv_heads: int, dim: int, vdim: int, positions: torch.Tensor,
                     seq_of: torch.Tensor, block_table: torch.Tensor, page: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                     q_out: torch.Tensor, write_kv: bool = True, err: Optional[torch.Tensor] = None,
                     stream: Optional[int] = None) -> None:
    """``qkv`` fp32 [T, q | k | v] (+ ``bias``): one RMS norm over the whole query projection (weight ``q_w`` of heads x
    dim) and one over the whole key projection, queries to ``q_out``, keys [.., dim] and values [.., vdim] to pages."""
    _check(qkv, "qkv", torch.float32)
    _check(q_out, "q_out")
    _check(k_pool, "k_pool", q_out.dtype)
    _check(v_pool, "v_pool", q_out.dtype)
    for t, n in ((positions, "positions"), (seq_of, "seq_of"), (block_table, "block_table")):
        _check(t, n, torch.int32)
    qn, kn, vn = heads * dim, kv_heads * dim, kv_heads * vdim
    for t, n, size in ((bias, "bias", qn + kn + vn), (q_w, "q_w", qn), (k_w, "k_w", kn)):
        if t is not None:
            _check(t, n, torch.float32)
            if t.numel() != size:
                raise KernelError(f"whole_norm_store: {n} has {t.numel()} elements, not {size}")
    _check_pages(k_pool, v_pool, kv_heads, page, dim, vdim, "whole_norm_store")
    if qkv.shape[0] < T or qkv.shape[1] < qn + kn + vn or q_out.numel() < T * qn:
        raise KernelError("whole_norm_store: buffers too small for the step")
    lib = _lib("sink_attention")
    _call(lib, lib.ember_whole_norm_store, _p(qkv), c_int(qkv.shape[1]), _p(bias), _p(q_w), _p(k_w), c_float(eps), c_int(T),
          c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), _p(positions), _p(seq_of), _p(block_table),
          c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), _p(q_out), _p(k_pool), _p(v_pool),
          c_int(dtype_code(q_out.dtype)), c_int(1 if write_kv else 0), _p(err), _stream(stream))


def latent_prepare(a: torch.Tensor, q_col: int, q_rank: int, c_col: int, kv_rank: int, rot_dim: int, q_w: Optional[torch.Tensor],
                   c_w: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rotary: int, T: int,
                   positions: torch.Tensor, seq_of: torch.Tensor, block_table: torch.Tensor, page: int, cq_out: Optional[torch.Tensor],
                   pool: Optional[torch.Tensor], write_kv: bool = True, err: Optional[torch.Tensor] = None,
                   stream: Optional[int] = None, half_layout: bool = False, magnitude: float = 1.0) -> None:
    """From the fused down-projections ``a`` fp32 [T, ld]: the query latent (columns q_col.., RMS norm with ``q_w``) to
    ``cq_out`` [T, q_rank] (none with q_rank 0); with ``write_kv`` the key/value latent (columns c_col.., RMS norm with
    ``c_w``) and behind it the shared key part (rot_dim columns, the first ``rotary`` rotated: neighbouring pairs, or
    element i with i + rotary / 2 under ``half_layout``; cosines and sines times ``magnitude``) into the token's cache
    row [kv_rank + rot_dim] of ``pool`` [pages, 1, page, kv_rank + rot_dim]."""
    _check(a, "a", torch.float32)
    if cq_out is None:
        if q_rank or pool is None:
            raise KernelError("latent_prepare: no output for the query latent")
        cq_out = pool                   # (only its type is read)
    _check(cq_out, "cq_out")
    for t, n in ((positions, "positions"), (seq_of, "seq_of"), (block_table, "block_table")):
        _check(t, n, torch.int32)
    for t, n in ((q_w, "q_w"), (c_w, "c_w"), (inv_freq, "inv_freq")):
        if t is not None:
            _check(t, n, torch.float32)
    if a.shape[0] < T or q_col + q_rank > a.shape[1] or cq_out.numel() < T * q_rank or (q_rank and (q_w is None or q_w.numel() != q_rank)):
        raise KernelError("latent_prepare: the query latent does not fit")
    if write_kv:
        _check(pool, "pool", cq_out.dtype)
        if c_col + kv_rank + rot_dim > a.shape[1] or c_w is None or c_w.numel() != kv_rank or \
                pool.dim() != 4 or tuple(pool.shape[1:]) != (1, page, kv_rank + rot_dim):
            raise KernelError("latent_prepare: the key/value latent does not fit its pages")
        if rotary and (inv_freq is None or inv_freq.numel() * 2 != rotary):
            raise KernelError(f"latent_prepare: frequencies for a rotation of {rotary}")
    lib = _lib("sink_attention")
    _call(lib, lib.ember_latent_prepare, _p(a), c_int(a.shape[1]), c_int(q_col), c_int(q_rank), c_int(c_col), c_int(kv_rank),
          c_int(rot_dim), _p(q_w), _p(c_w), c_float(eps), _p(inv_freq), c_int(rotary if write_kv else 0), c_int(T), _p(positions),
          _p(seq_of), _p(block_table), c_int(block_table.shape[-1]), c_int(page), c_int(pool.shape[0] if pool is not None else 1),
          _p(cq_out), _p(pool), c_int(dtype_code(cq_out.dtype)), c_int(1 if write_kv else 0), c_int(1 if half_layout else 0),
          c_float(magnitude), _p(err), _stream(stream))


def rotate_pairs(x: torch.Tensor, x_head: int, x_col: int, out: torch.Tensor, out_head: int, out_col: int, T: int, heads: int,
                 width: int, rotary: int, inv_freq: Optional[torch.Tensor], positions: torch.Tensor,
                 stream: Optional[int] = None, half_layout: bool = False, magnitude: float = 1.0) -> None:
    """out[t, h, out_col + i] = x[t, h, x_col + i] for i < width, with pairs (2i, 2i + 1) (under ``half_layout``:
    (i, i + rotary / 2)) below ``rotary`` turned by float(position) * inv_freq[i], cosine and sine times ``magnitude``;
    x fp32 rows of heads ``x_head`` apart, out rows of heads ``out_head`` apart."""
    _check(x, "x", torch.float32)
    _check(out, "out")
    _check(positions, "positions", torch.int32)
    if inv_freq is not None:
        _check(inv_freq, "inv_freq", torch.float32)
    if rotary and (inv_freq is None or inv_freq.numel() * 2 != rotary):
        raise KernelError(f"rotate_pairs: frequencies for a rotation of {rotary}")
    if x.shape[0] < T or out.shape[0] < T or (heads - 1) * x_head + x_col + width > x.shape[1] or \
            (heads - 1) * out_head + out_col + width > out.shape[1]:
        raise KernelError("rotate_pairs: the slices do not fit their rows")
    lib = _lib("sink_attention")
    _call(lib, lib.ember_rotate_pairs, _p(x), c_int(x.shape[1]), c_int(x_head), c_int(x_col), _p(out), c_int(out.shape[1]),
          c_int(out_head), c_int(out_col), c_int(dtype_code(out.dtype)), c_int(T), c_int(heads), c_int(width), c_int(rotary),
          _p(inv_freq), _p(positions), c_int(1 if half_layout else 0), c_float(magnitude), _stream(stream))


def head_gemm(x: torch.Tensor, x_head: int, x_col: int, w: torch.Tensor, out: torch.Tensor, out_head: int, out_col: int, T: int,
              gate: Optional[torch.Tensor] = None, gate_col: int = 0, stream: Optional[int] = None) -> None:
    """out[t, h, out_col + n] = sum_k x[t, h, x_col + k] * w[h, n, k], a product per head (``w`` [heads, N, K]); with
    ``gate`` (fp32 rows) the result is multiplied by sigmoid(gate[t, gate_col + h N + n]).  x fp32 2-D."""
    _check(x, "x", torch.float32)
    _check(w, "w")
    _check(out, "out")
    H, N, K = w.shape
    if x.shape[0] < T or out.shape[0] < T or (H - 1) * x_head + x_col + K > x.shape[1] or (H - 1) * out_head + out_col + N > out.shape[1]:
        raise KernelError(f"head_gemm: {H} heads of {N} x {K} do not fit rows of {x.shape[1]} -> {out.shape[1]}")
    if gate is not None:
        _check(gate, "gate", torch.float32)
        if gate.shape[0] < T or gate_col + H * N > gate.shape[1]:
            raise KernelError("head_gemm: the gate does not fit")
    lib = _lib("sink_attention")
    _call(lib, lib.ember_head_gemm, _p(x), c_int(x.shape[1]), c_int(x_head), c_int(x_col), _p(w), c_int(dtype_code(w.dtype)), _p(out),
          c_int(dtype_code(out.dtype)), c_int(out.shape[1]), c_int(out_head), c_int(out_col), _p(gate),
          c_int(gate.shape[1] if gate is not None else 0), c_int(gate_col), c_int(T), c_int(H), c_int(N), c_int(K), _stream(stream))


def sink_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: Optional[torch.Tensor], out: torch.Tensor, T: int, heads: int,
                   kv_heads: int, dim: int, vdim: int, tiles: torch.Tensor, n_tiles: int, tile_q: int, block_table: torch.Tensor,
                   page: int, window: int, keep_first: int, sink: Optional[torch.Tensor], scale: float, n_splits: int = 1,
                   split_keys: int = 0, part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                   err: Optional[torch.Tensor] = None, stream: Optional[int] = None, chunk: int = 0,
                   softcap: float = 0.0, head_gate: Optional[torch.Tensor] = None, head_gate_col: int = 0) -> None:
    """out[t, h] = sum_j w_j v_j over the visible keys j <= t (under a window: t - j < window or j < keep_first), w the
    softmax of scale * q . k_j whose denominator also holds exp(sink[h]).  Keys [.., dim], values [.., vdim]; without
    ``v_pool`` a value is the first ``vdim`` elements of the key row.  ``out`` is q's dtype or float32.  ``chunk`` > 0:
    j is visible only if floor(t / chunk) == floor(j / chunk) (positions, counted from the sequence's start);
    ``softcap`` > 0: the scaled score becomes softcap * tanh(score / softcap); ``head_gate`` (fp32 [T, >= heads] logits):
    head h's output is multiplied by sigmoid(head_gate[t, head_gate_col + h])."""
    _check_head_gate(head_gate, T, heads, head_gate_col)
    _check(q, "q")
    _check(k_pool, "k_pool", q.dtype)
    if v_pool is not None:
        _check(v_pool, "v_pool", q.dtype)
    _check(out, "out")
    if out.dtype not in (q.dtype, torch.float32):
        raise KernelError(f"sink_attention: output {out.dtype} for queries {q.dtype}")
    _check(tiles, "tiles", torch.int32)
    _check(block_table, "block_table", torch.int32)
    if sink is not None:
        _check(sink, "sink", torch.float32)
        if sink.numel() != heads:
            raise KernelError(f"sink_attention: {sink.numel()} sinks for {heads} heads")
    _check_pages(k_pool, v_pool, kv_heads, page, dim, vdim, "sink_attention")
    if q.numel() < T * heads * dim or out.numel() < T * heads * vdim:
        raise KernelError("sink_attention: q/out too small for the step")
    if n_splits > 1:
        _check(part_o, "part_o", torch.float32)
        _check(part_ml, "part_ml", torch.float32)
        if part_o.numel() < T * heads * n_splits * vdim or part_ml.numel() < T * heads * n_splits * 2:
            raise KernelError("sink_attention: split buffers too small")
    lib = _lib("sink_attention")
    _call(lib, lib.ember_sink_attention, _p(q), _p(k_pool), _p(v_pool), _p(out), c_int(dtype_code(q.dtype)),
          c_int(1 if out.dtype == torch.float32 else 0), c_int(T), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), _p(tiles),
          c_int(n_tiles), c_int(tile_q), _p(block_table), c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]),
          c_int(window), c_int(keep_first), _p(sink), c_float(scale), c_int(n_splits), c_int(split_keys), _p(part_o), _p(part_ml),
          _p(err), c_int(chunk), c_float(softcap), (_off(head_gate, head_gate_col) if head_gate is not None else _p(None)), c_int(head_gate.shape[-1] if head_gate is not None else 0),
          _stream(stream))


# --------------------------------------------------------------------- routed feed-forward (csrc/moe.cu)
MOE_TILE_ROWS = 32               # slots of one expert a block of the tiled products takes (its MOE_BM)
MOE_STREAM_ROWS = 16             # ... and a block of the streaming products (its MS_ROWS)
MOE_MAX_EXPERTS, MOE_MAX_TOP = 256, 32


def moe_max_tiles(n_pairs: int, experts: int, tile_rows: int = MOE_TILE_ROWS) -> int:
    """The most row tiles a step of ``n_pairs`` (token, choice) pairs can have: every expert may end in a ragged tile."""
    return n_pairs // tile_rows + experts


def moe_stream_usable(x: torch.Tensor, K: int) -> bool:
    """Whether the streaming products take rows of ``K`` elements of x's type: multiples of 16 bytes, 16 of them in
    shared memory."""
    return (K * x.element_size()) % 16 == 0 and MOE_STREAM_ROWS * K * x.element_size() <= 200 * 1024


def _route_rule(rule, experts: int):
    """(sigmoid, correction pointer, scale, renormalize) of a routing rule: None is the softmax over the chosen logits;
    else (correction fp32 [experts] or None, scale, renormalize) for sigmoid scores."""
    if rule is None:
        return c_int(0), c_void_p(0), c_float(1.0), c_int(0), c_int(0), c_int(0)
    correction, scale, renormalize = rule[:3]
    # longer rules: (..., scoring, groups, keep) with scoring "sigmoid" or "softmax" (over all experts) and the choice
    # limited to the ``keep`` best of ``groups`` equal groups of neighbouring experts (groups 0: no limit)
    scoring, groups, keep = (tuple(rule[3:]) + ("sigmoid", 0, 0)[len(rule) - 3:]) if len(rule) > 3 else ("sigmoid", 0, 0)
    if scoring not in ("sigmoid", "softmax"):
        raise KernelError(f"routing: scoring {scoring!r}")
    if groups and (groups > 32 or experts % groups or not 1 <= keep <= groups):
        raise KernelError(f"routing: {groups} groups (at most 32, dividing {experts} experts) of which {keep} are kept")
    if correction is not None:
        _check(correction, "correction", torch.float32)
        if correction.numel() != experts:
            raise KernelError(f"routing: a correction of {correction.numel()} for {experts} experts")
    return (c_int(1 if scoring == "sigmoid" else 2), _p(correction), c_float(scale), c_int(1 if renormalize else 0), c_int(groups),
            c_int(keep))


def moe_route(logits: torch.Tensor, T: int, top: int, sel: torch.Tensor, wgt: torch.Tensor, stream: Optional[int] = None,
              rule=None) -> None:
    """sel[t] = the ``top`` experts with the largest logits (descending; ties: the lower index), wgt[t] = softmax over
    those logits alone.  logits fp32 [T, experts].  With ``rule`` = (correction, scale, renormalize): scores are
    sigmoid(logits), the choice is by score + correction, the weights are the chosen scores times scale (divided by
    their sum first if renormalize)."""
    _check(logits, "logits", torch.float32)
    _check(sel, "sel", torch.int32)
    _check(wgt, "wgt", torch.float32)
    if logits.dim() != 2 or logits.shape[0] < T or sel.numel() < T * top or wgt.numel() < T * top:
        raise KernelError("moe_route: buffers do not fit the step")
    lib = _lib("moe")
    _call(lib, lib.ember_moe_route, _p(logits), c_int(T), c_int(logits.shape[1]), c_int(top), _p(sel), _p(wgt),
          *_route_rule(rule, logits.shape[1]), _stream(stream))


def moe_group(sel: torch.Tensor, n_pairs: int, experts: int, offsets: torch.Tensor, pair_of_slot: torch.Tensor,
              slot_of_pair: torch.Tensor, tiles: torch.Tensor, tile_rows: int = MOE_TILE_ROWS, stream: Optional[int] = None,
              tiled: int = 0) -> int:
    """Orders the (token, choice) pairs by expert.  offsets int32 [experts + 1]; pair_of_slot, slot_of_pair int32
    [n_pairs]; tiles int32 [1 + 2 max_tiles]: the number of row tiles (of up to ``tile_rows`` slots of one expert),
    then every tile's expert, then every tile's first slot.  Returns max_tiles (what the products' grids are sized for).
    ``tiled`` > 0: only the first ``tiled`` experts have weights; the others' pairs get slots but no tiles."""
    for t, n in ((sel, "sel"), (offsets, "offsets"), (pair_of_slot, "pair_of_slot"), (slot_of_pair, "slot_of_pair"), (tiles, "tiles")):
        _check(t, n, torch.int32)
    mt = moe_max_tiles(n_pairs, experts, tile_rows)
    if sel.numel() < n_pairs or offsets.numel() < experts + 1 or pair_of_slot.numel() < n_pairs or slot_of_pair.numel() < n_pairs or \
            tiles.numel() < 1 + 2 * mt:
        raise KernelError("moe_group: buffers do not fit the step")
    lib = _lib("moe")
    _call(lib, lib.ember_moe_group, _p(sel), c_int(n_pairs), c_int(experts), _p(offsets), _p(pair_of_slot), _p(slot_of_pair),
          _off(tiles, 0), _off(tiles, 1), _off(tiles, 1 + mt), c_int(mt), c_int(tile_rows), c_int(tiled), _stream(stream))
    return mt


def moe_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor, pair_of_slot: torch.Tensor,
             tiles: torch.Tensor, max_tiles: int, top: int, gated: bool, limit: float = 0.0, alpha: float = 1.0,
             stream: Optional[int] = None, streaming: bool = False, up_offset: float = 1.0, square_relu: bool = False) -> None:
    """The product of every slot's row with its expert's matrix (``w`` [experts, N, K]).  ``top`` > 0: a slot's row of
    ``x`` is its token's (x [tokens, K], gathered through the pairs); 0: x has a row per slot.  ``gated``: w's rows are
    interleaved (gate, up) and out[slot, j] = g sigmoid(alpha g) (u + up_offset) with g = min(gate, limit),
    u = clamp(up, -limit, limit) (``limit`` may be infinite), in x's dtype; else out[slot] is the fp32 product, or with
    ``square_relu`` relu(product)^2 in x's dtype (an ungated expert's activation).  ``streaming``: the form for tile
    lists of 16-row tiles (``moe_group`` with ``MOE_STREAM_ROWS``), else the form for 32-row tiles."""
    _check(x, "x")
    _check(w, "w", x.dtype)
    if gated and square_relu:
        raise KernelError("moe_gemm: relu^2 is the activation of an ungated product")
    _check(out, "out", x.dtype if (gated or square_relu) else torch.float32)
    E, N, K = w.shape
    n_out = N // 2 if gated else N
    if x.shape[-1] != K or out.shape[-1] != n_out:
        raise KernelError(f"moe_gemm: rows of {x.shape[-1]} -> {out.shape[-1]} against experts {tuple(w.shape)}")
    lib = _lib("moe")
    _call(lib, lib.ember_moe_stream if streaming else lib.ember_moe_gemm, _p(x), c_int(dtype_code(x.dtype)), c_int(K), _p(w), c_int(dtype_code(w.dtype)), c_longlong(N * K),
          _p(out), c_int(dtype_code(out.dtype)), c_int(n_out), _p(offsets), _p(pair_of_slot), _off(tiles, 0), _off(tiles, 1),
          _off(tiles, 1 + max_tiles), c_int(max_tiles), c_int(top), c_int(N), c_int(K), c_int(1 if gated else 0), c_float(limit),
          c_float(alpha), c_float(up_offset), c_int(1 if square_relu else 0), _stream(stream))


def moe_combine(y: torch.Tensor, wgt: torch.Tensor, slot_of_pair: torch.Tensor, T: int, top: int, out: torch.Tensor,
                accumulate: bool = False, stream: Optional[int] = None, sel: Optional[torch.Tensor] = None, experts: int = 0,
                same: Optional[torch.Tensor] = None) -> None:
    """out[t] (+)= sum over the token's choices, in order, of wgt[t, k] * y[slot of (t, k)]; all fp32.  With ``sel``
    (the choices) a choice from ``experts`` on is an identity expert, whose output is the token's row of ``same``
    (fp32 or bfloat16 [T, hidden]) instead of a row of y."""
    _check(y, "y", torch.float32)
    _check(wgt, "wgt", torch.float32)
    _check(out, "out", torch.float32)
    _check(slot_of_pair, "slot_of_pair", torch.int32)
    hidden = out.shape[-1]
    if y.shape[-1] != hidden or y.numel() < T * top * hidden or out.numel() < T * hidden:
        raise KernelError("moe_combine: buffers do not fit the step")
    if sel is not None:
        _check(sel, "sel", torch.int32)
        _check(same, "same")
        if same.dtype not in (torch.float32, torch.bfloat16) or same.shape[-1] != hidden or same.numel() < T * hidden or sel.numel() < T * top:
            raise KernelError("moe_combine: the identity experts' rows do not fit the step")
    lib = _lib("moe")
    _call(lib, lib.ember_moe_combine, _p(y), _p(wgt), _p(slot_of_pair), c_int(T), c_int(top), _p(out), c_int(1 if accumulate else 0),
          c_int(hidden), _p(sel), c_int(experts), _p(same if sel is not None else None),
          c_int(dtype_code(same.dtype) if sel is not None else 0), _stream(stream))


def moe_gather(x: torch.Tensor, pair_of_slot: torch.Tensor, n_pairs: int, top: int, xs: torch.Tensor, stream: Optional[int] = None) -> None:
    """xs[slot] = x[token of the slot's pair]: every expert's rows side by side (rows of a multiple of 16 bytes)."""
    _check(x, "x")
    _check(xs, "xs", x.dtype)
    _check(pair_of_slot, "pair_of_slot", torch.int32)
    row = x.shape[-1] * x.element_size()
    if xs.shape[-1] != x.shape[-1] or xs.numel() < n_pairs * x.shape[-1] or pair_of_slot.numel() < n_pairs:
        raise KernelError("moe_gather: buffers do not fit the step")
    lib = _lib("moe")
    _call(lib, lib.ember_moe_gather, _p(x), _p(pair_of_slot), c_int(n_pairs), c_int(top), _p(xs), c_int(row), _stream(stream))


def moe_activation(gu: torch.Tensor, act: torch.Tensor, rows: int, limit: float, alpha: float, stream: Optional[int] = None,
                   up_offset: float = 1.0, bias: Optional[torch.Tensor] = None) -> None:
    """act[r, j] = g sigmoid(alpha g) (u + up_offset) with g = min(gu[r, 2j], limit), u = clamp(gu[r, 2j + 1], -limit, limit); gu fp32.
    ``bias`` (fp32 [2n], interleaved like a row of gu) is added to gu first."""
    _check(gu, "gu", torch.float32)
    _check(act, "act")
    n = act.shape[-1]
    if gu.shape[-1] != 2 * n or gu.numel() < rows * 2 * n or act.numel() < rows * n:
        raise KernelError("moe_activation: buffers do not fit")
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != 2 * n:
            raise KernelError("moe_activation: the biases do not fit the rows")
    lib = _lib("moe")
    _call(lib, lib.ember_moe_activation, _p(gu), _p(act), c_int(dtype_code(act.dtype)), c_longlong(rows * n), c_float(limit),
          c_float(alpha), c_float(up_offset), _p(bias), c_int(n), _stream(stream))


def moe_square_relu(x: torch.Tensor, act: torch.Tensor, n: int, stream: Optional[int] = None) -> None:
    """act[:n] = relu(x[:n])^2 (x fp32): the activation of an ungated expert whose product left fp32 sums."""
    _check(x, "x", torch.float32)
    _check(act, "act")
    if x.numel() < n or act.numel() < n:
        raise KernelError("moe_square_relu: buffers do not fit")
    lib = _lib("moe")
    _call(lib, lib.ember_moe_square_relu, _p(x), _p(act), c_int(dtype_code(act.dtype)), c_longlong(n), _stream(stream))


def moe_router(x: torch.Tensor, w: torch.Tensor, T: int, top: int, sel: torch.Tensor, wgt: torch.Tensor,
               logits: Optional[torch.Tensor] = None, stream: Optional[int] = None, rule=None) -> None:
    """The router's logits x[t] . w[e] (``w`` fp32 [experts, K], fp32 sums) and ``moe_route`` on them (with its
    ``rule``) in one kernel; ``logits`` (fp32 [T, experts]) receives them if given."""
    _check(x, "x")
    _check(w, "w", torch.float32)
    _check(sel, "sel", torch.int32)
    _check(wgt, "wgt", torch.float32)
    E, K = w.shape
    if x.shape[-1] != K or x.numel() < T * K or sel.numel() < T * top or wgt.numel() < T * top:
        raise KernelError("moe_router: buffers do not fit the step")
    if logits is not None:
        _check(logits, "logits", torch.float32)
        if logits.numel() < T * E:
            raise KernelError("moe_router: the logits do not fit")
    lib = _lib("moe")
    _call(lib, lib.ember_moe_router, _p(x), c_int(dtype_code(x.dtype)), _p(w), c_int(T), c_int(K), c_int(E), c_int(top), _p(sel),
          _p(wgt), _p(logits), *_route_rule(rule, E), _stream(stream))


SHARED_ROW_TC_ROWS = 64          # (query, head) rows of a block of the tensor-core form (its LT_ROWS)


def shared_row_attention_tc_usable(q: torch.Tensor, v_pool, dim: int, vdim: int) -> bool:
    """Whether the tensor-core form of ``sink_attention`` takes this layout: bfloat16, head sizes that are multiples
    of 16 (with or without a value pool)."""
    return (TC_ENABLED and q.dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 and vdim <= 512
            and (v_pool is not None or vdim <= dim)
            and ((SHARED_ROW_TC_ROWS + 64) * (dim + 8) + (64 * (vdim + 8) if v_pool is not None else 0)) * 2 <= 220 * 1024)


def shared_row_attention_tc_tile_queries(group: int) -> int:
    return max(1, SHARED_ROW_TC_ROWS // max(1, min(group, SHARED_ROW_TC_ROWS)))


def shared_row_attention_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: Optional[torch.Tensor], out: torch.Tensor, T: int, heads: int, kv_heads: int, dim: int,
                            vdim: int, tiles: torch.Tensor, n_tiles: int, tile_q: int, block_table: torch.Tensor, page: int,
                            window: int, keep_first: int, sink: Optional[torch.Tensor], scale: float, n_splits: int = 1,
                            split_keys: int = 0, part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                            err: Optional[torch.Tensor] = None, stream: Optional[int] = None, chunk: int = 0,
                   softcap: float = 0.0, head_gate: Optional[torch.Tensor] = None, head_gate_col: int = 0) -> None:
    """``sink_attention`` on the tensor cores (bfloat16 queries, keys, values; scores, weights and sums fp32)."""
    _check_head_gate(head_gate, T, heads, head_gate_col)
    _check(q, "q", torch.bfloat16)
    _check(k_pool, "k_pool", torch.bfloat16)
    if v_pool is not None:
        _check(v_pool, "v_pool", torch.bfloat16)
    _check(out, "out")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"shared_row_attention_tc: output {out.dtype}")
    _check(tiles, "tiles", torch.int32)
    _check(block_table, "block_table", torch.int32)
    if sink is not None:
        _check(sink, "sink", torch.float32)
        if sink.numel() != heads:
            raise KernelError(f"shared_row_attention_tc: {sink.numel()} sinks for {heads} heads")
    _check_pages(k_pool, v_pool, kv_heads, page, dim, vdim, "shared_row_attention_tc")
    if q.numel() < T * heads * dim or out.numel() < T * heads * vdim:
        raise KernelError("shared_row_attention_tc: q/out too small for the step")
    if n_splits > 1:
        _check(part_o, "part_o", torch.float32)
        _check(part_ml, "part_ml", torch.float32)
        if part_o.numel() < T * heads * n_splits * vdim or part_ml.numel() < T * heads * n_splits * 2:
            raise KernelError("shared_row_attention_tc: split buffers too small")
    lib = _lib("sink_attention")
    _call(lib, lib.ember_shared_row_attention_tc, _p(q), _p(k_pool), _p(v_pool), _p(out), c_int(1 if out.dtype == torch.float32 else 0), c_int(T),
          c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), _p(tiles), c_int(n_tiles), c_int(tile_q), _p(block_table),
          c_int(block_table.shape[-1]), c_int(page), c_int(k_pool.shape[0]), c_int(window), c_int(keep_first), _p(sink),
          c_float(scale), c_int(n_splits), c_int(split_keys), _p(part_o), _p(part_ml), _p(err), c_int(chunk), c_float(softcap),
          (_off(head_gate, head_gate_col) if head_gate is not None else _p(None)), c_int(head_gate.shape[-1] if head_gate is not None else 0), _stream(stream))
