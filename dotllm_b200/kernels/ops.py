"""Tensor-level wrappers of the CUDA kernels.

Each function checks devices, dtypes, shapes and strides on the host, then launches on
the current CUDA stream.  Tensors that are not on a CUDA device are refused: there is no
CPU path.  Parts call these functions through the module (``ops.add_rmsnorm(...)``).
"""
from __future__ import annotations

import torch

from ..errors import KernelError
from . import attention_fast, gemm_skinny, gemm_tc
from . import library as _library

PAGE = 64                      # tokens per cache page (DL_PAGE in csrc/common.cuh)
_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


def _code(dtype):
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _stream():
    return _library.current_stream()


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only: there is no CPU fallback")
    _library.require_device()


def _ptr(t):
    return None if t is None else t.data_ptr()


def _rows_view(t, what):
    """A 2-D tensor whose rows are contiguous (a column slice of a wider matrix is fine)."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: need a 2-D tensor with contiguous rows, got shape "
                          f"{tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _int32(t, what):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what}: need a contiguous int32 tensor")
    return t


# ------------------------------------------------------------------ embedding
def gather_rows(table, ids, out=None, out_dtype=torch.float32):
    """out[r] = table[ids[r]] as ``out_dtype``.  table [n, width] float32 or bfloat16 (rows contiguous,
    possibly with gaps between them); ids int32 [R]; float32 out, or bfloat16 from a bfloat16 table."""
    _need_cuda(table, ids, out)
    stride = _rows_view(table, "gather_rows table")
    _int32(ids, "gather_rows ids")
    n, width = table.shape
    rows = ids.numel()
    if out is None:
        out = torch.empty((rows, width), dtype=out_dtype, device=table.device)
    elif out.shape != (rows, width) or out.dtype != out_dtype or not out.is_contiguous():
        raise KernelError(f"gather_rows: out must be contiguous {out_dtype} [rows, width]")
    if out_dtype != torch.float32 and out_dtype != table.dtype:
        raise KernelError(f"gather_rows: rows of {table.dtype} are gathered as float32 or as they are, not as {out_dtype}")
    _library.call("dl_gather_rows", _ptr(table), _code(table.dtype), stride, _ptr(ids), _ptr(out), _code(out_dtype),
                  rows, width, n, _stream())
    return out


# ------------------------------------------------- products not yet launched
class PendingProduct:
    """x W^T (float32 result of bfloat16 operands) that ``linear(..., lazy=True)`` has not launched
    yet.  Given to ``add_rmsnorm`` as the delta, the product itself adds its result into the stream
    (the decode kernels in their epilogue, the library product as its accumulate operand); anyone
    else calls ``tensor()`` (or ``resolve``) and gets the plain float32 product."""

    def __init__(self, x, w, resident):
        self.x, self.w, self.resident = x, w, resident
        self.shape = (x.shape[0], w.shape[0])

    def tensor(self):
        return linear(self.x, self.w, out_dtype=torch.float32, resident=self.resident)

    def add_into(self, residual):
        """residual += x W^T by the library product with the stream as its accumulate operand (one
        rounding of accumulator + stream, as the separate addition has; no [T, N] product is
        written and read back).  False when the sizes belong to the decode kernels or the
        tensors do not fit; nothing has happened then."""
        x = self.x
        if isinstance(x, ScaledRows) or x.dtype != torch.bfloat16 or not x.is_cuda or x.dim() != 2 \
                or residual.dtype != torch.float32 or not residual.is_contiguous() \
                or tuple(residual.shape) != self.shape or gemm_skinny.takes(x, self.w):
            return False
        torch.addmm(residual, x, self.w.t(), out_dtype=torch.float32, out=residual)
        return True


class ScaledRows:
    """A normalised stream still lacking its factor per row: ``data`` = stream * gain (bfloat16) and the
    sums of squares per part of 16 (the mma.sync product's) or 128 columns (the tcgen05 product's), left by the product that added into the stream.  ``linear``
    and ``gated_linear`` take it as x and apply rsqrt(mean + eps) to their output rows - the product
    of the normalised rows, since the factor is one number per row.  ``tensor()`` gives the
    normalised rows themselves (valid until the stream is added to again)."""

    def __init__(self, data, sums, width, eps, stream, gain):
        self.data, self.sums, self.width, self.eps = data, sums, width, eps
        self.stream, self.gain = stream, gain
        self.shape, self.dtype = data.shape, data.dtype

    def row_sums(self):
        return self.sums, self.sums.numel() // gemm_skinny.sum_stride(self.data.shape[0]), self.width, self.eps

    def tensor(self):
        return add_rmsnorm(self.stream, None, self.gain, self.eps, self.data.dtype)


def resolve(value):
    """The tensor behind a PendingProduct or ScaledRows; tensors and None pass through."""
    return value.tensor() if isinstance(value, (PendingProduct, ScaledRows)) else value


def narrow_rows(value, ids):
    """The rows ``ids`` (int32 on the device) of a branch output, in its own dtype.  Of a product not
    yet launched only those rows of x are kept, so that the product is computed for them alone."""
    if value is None:
        return None
    if isinstance(value, PendingProduct):
        x = resolve(value.x)
        return PendingProduct(gather_rows(x, ids, out_dtype=x.dtype), value.w, value.resident)
    value = resolve(value)
    return gather_rows(value, ids, out_dtype=value.dtype)


# ----------------------------------------------------------------------- norm
def add_rmsnorm(residual, delta, gain, eps, out_dtype, lazy=False):
    """residual += delta (when delta is given), then rmsnorm(residual) * gain in ``out_dtype``.

    residual: float32 [T, H] contiguous, updated in place.  delta: [T, H] float32/bfloat16, a
    PendingProduct, or None.  gain: float32 [H].  ``lazy``: the caller will hand the result straight
    to ``linear`` / ``gated_linear``, so it may be a ScaledRows: a pending product then does the
    addition itself and the next product the normalisation, with no kernel in between."""
    if isinstance(delta, PendingProduct):
        fused = _add_product_scaled(residual, delta, gain, eps, out_dtype) if lazy else None
        if fused is not None:
            return fused
        delta = None if delta.add_into(residual) else delta.tensor()
    _need_cuda(residual, delta, gain)
    if residual.dtype != torch.float32 or residual.dim() != 2 or not residual.is_contiguous():
        raise KernelError("rmsnorm: the residual stream must be contiguous float32 [T, H]")
    rows, width = residual.shape
    if gain.dtype != torch.float32 or gain.shape != (width,) or not gain.is_contiguous():
        raise KernelError(f"rmsnorm: gain must be float32 [{width}]")
    if delta is not None and (delta.shape != residual.shape or not delta.is_contiguous()):
        raise KernelError("rmsnorm: delta must be contiguous with the residual's shape")
    out = torch.empty((rows, width), dtype=out_dtype, device=residual.device)
    _library.call("dl_add_rmsnorm", _ptr(residual), _ptr(delta),
                  _code(delta.dtype) if delta is not None else 0, _ptr(gain), _ptr(out),
                  _code(out_dtype), rows, width, float(eps), _stream())
    return out


def _add_product_scaled(residual, product, gain, eps, out_dtype):
    x = product.x
    rows = x.row_sums() if isinstance(x, ScaledRows) else None
    xt = x.data if rows is not None else x
    if out_dtype != torch.bfloat16 or residual.dtype != torch.float32 or residual.dim() != 2 \
            or residual.stride(1) != 1 or tuple(residual.shape) != product.shape \
            or gain.dtype != torch.float32 or gain.shape != (residual.shape[1],) or not gain.is_contiguous() \
            or not gemm_skinny.takes(xt, product.w):
        return None
    _need_cuda(residual, xt, product.w, gain)
    scaled, sums = gemm_skinny.run(xt, product.w, torch.float32, resident=product.resident, row_sums=rows,
                                   into=(residual, gain))
    return ScaledRows(scaled, sums, residual.shape[1], eps, residual, gain)


# --------------------------------------------------- position + cache write
def rope_cache_write(q, k, v, cos, sin, rotary_dim, token_seq, token_pos, block_table,
                     k_pool, v_pool, n_heads, n_kv_heads, head_dim, write_cache=True):
    """Rotate Q in place (and K on its way into the cache); store K and V at each token's page.

    q [T, nh*hd], k, v [T, nkv*hd]: row-contiguous views of one dtype.  cos, sin: float32
    [positions, rotary_dim/2] (None with rotary_dim 0: no rotation).  k_pool [pages, nkv, 64, hd],
    v_pool [pages, nkv, hd, 64].  block_table int32 [B, P]; token_seq/token_pos int32 [T]."""
    _need_cuda(q, k, v, cos, sin, token_seq, token_pos, block_table, k_pool, v_pool)
    T = q.shape[0]
    qs = _rows_view(q, "rope q")
    if q.shape[1] != n_heads * head_dim:
        raise KernelError("rope: q width is not n_heads * head_dim")
    ks = vs = 0
    n_pages = 0
    bt_stride = 0
    if write_cache:
        ks = _rows_view(k, "rope k")
        vs = _rows_view(v, "rope v")
        if k.shape != (T, n_kv_heads * head_dim) or v.shape != k.shape:
            raise KernelError("rope: k and v must be [T, n_kv_heads * head_dim]")
        if k.dtype != q.dtype or v.dtype != q.dtype or k_pool.dtype != q.dtype or v_pool.dtype != q.dtype:
            raise KernelError("rope: q, k, v and the cache must share one dtype")
        n_pages = _check_pools(k_pool, v_pool, n_kv_heads, head_dim)
        _int32(block_table, "block_table")
        bt_stride = block_table.shape[1]
        _int32(token_seq, "token_seq")
    _int32(token_pos, "token_pos")
    table_rows = 0
    if rotary_dim:
        if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != sin.shape \
                or cos.dim() != 2 or cos.shape[1] != rotary_dim // 2 or not cos.is_contiguous() \
                or not sin.is_contiguous():
            raise KernelError("rope: cos/sin must be contiguous float32 [positions, rotary_dim/2]")
        table_rows = cos.shape[0]
    _library.call("dl_rope_cache_write", _ptr(q), qs, _ptr(k) if write_cache else None, ks,
                  _ptr(v) if write_cache else None, vs, _code(q.dtype),
                  _ptr(cos) if rotary_dim else None, _ptr(sin) if rotary_dim else None,
                  int(rotary_dim), table_rows, _ptr(token_seq) if write_cache else None, _ptr(token_pos),
                  _ptr(block_table) if write_cache else None, bt_stride,
                  _ptr(k_pool) if write_cache else None, _ptr(v_pool) if write_cache else None, n_pages,
                  T, n_heads, n_kv_heads, head_dim, 1 if write_cache else 0, _stream())


def _check_pools(k_pool, v_pool, n_kv_heads, head_dim):
    if k_pool.dim() != 4 or not k_pool.is_contiguous() or not v_pool.is_contiguous() \
            or tuple(k_pool.shape[1:]) != (n_kv_heads, PAGE, head_dim) \
            or tuple(v_pool.shape) != (k_pool.shape[0], n_kv_heads, head_dim, PAGE):
        raise KernelError(f"cache pools must be K [pages, {n_kv_heads}, {PAGE}, {head_dim}] and "
                          f"V [pages, {n_kv_heads}, {head_dim}, {PAGE}], got {tuple(k_pool.shape)} "
                          f"and {tuple(v_pool.shape)}")
    return k_pool.shape[0]


# ------------------------------------------------------------------ attention
class ScoreHook:
    """A change of the attention scores before the softmax: ``softcap`` > 0 turns a score s into
    softcap * tanh(s / softcap); ``slopes`` (float32 [n_heads] on the device) then adds
    slope * (key position - query position).  Only the generic kernel honours a hook: the
    tensor-core kernels take none, so a mixer that sets one runs on the generic kernel."""

    def __init__(self, softcap=0.0, slopes=None):
        self.softcap = float(softcap)
        self.slopes = slopes
        if self.softcap < 0:
            raise KernelError("a score hook's softcap must be 0 (none) or positive")

    def __bool__(self):
        return self.softcap > 0 or self.slopes is not None


def attention(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads,
              head_dim, scale, window=0, plan=None, score_hook=None):
    """Causal attention of the step's tokens over their sequences' cached keys and values.

    q [T, nh*hd] (row-contiguous view); returns [T, nh*hd] of q's dtype.  ``window`` 0 means
    every earlier key; w > 0 means the last w keys.  ``plan`` carries the per-step layout
    (sequence lengths, chunking) that the tensor-core kernels need; without one, for sizes
    they do not take, or with a ``score_hook``, the generic kernel runs."""
    _need_cuda(q, k_pool, v_pool, token_seq, token_pos, block_table)
    T = q.shape[0]
    qs = _rows_view(q, "attention q")
    if q.shape[1] != n_heads * head_dim:
        raise KernelError("attention: q width is not n_heads * head_dim")
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype:
        raise KernelError("attention: q and the cache must share one dtype")
    n_pages = _check_pools(k_pool, v_pool, n_kv_heads, head_dim)
    _int32(token_seq, "token_seq")
    _int32(token_pos, "token_pos")
    _int32(block_table, "block_table")
    out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    softcap, slopes = 0.0, None
    if score_hook:
        softcap, slopes = score_hook.softcap, score_hook.slopes
        if slopes is not None and (slopes.dtype != torch.float32 or slopes.shape != (n_heads,) or not slopes.is_contiguous()
                                   or not slopes.is_cuda):
            raise KernelError(f"attention: a score hook's slopes must be contiguous float32 [{n_heads}] on the device")
    if plan is not None and q.dtype == torch.bfloat16 and not score_hook:
        if attention_fast.run(q, qs, out, k_pool, v_pool, n_pages, token_seq, token_pos, block_table,
                              n_heads, n_kv_heads, head_dim, float(scale), int(window), plan):
            return out
    _library.call("dl_attention_generic", _ptr(q), qs, _ptr(out), out.stride(0), _code(q.dtype),
                  _ptr(k_pool), _ptr(v_pool), n_pages, _ptr(token_seq), _ptr(token_pos),
                  _ptr(block_table), block_table.shape[1], T, n_heads, n_kv_heads, head_dim,
                  float(scale), int(window), float(softcap), _ptr(slopes), _stream())
    return out


def rope_cache_attention(q, k, v, cos, sin, rotary_dim, token_seq, token_pos, block_table, k_pool, v_pool,
                         n_heads, n_kv_heads, head_dim, scale, window=0, plan=None, score_hook=None):
    """``rope_cache_write`` followed by ``attention`` (same arguments, same result).  A bfloat16
    decode step (one new token per sequence) with a full-width rotation of head size 64 or 128, or
    with no rotation, runs as one kernel that rotates q, puts the new keys and values into the
    cache and attends; everything else runs the two kernels one after the other."""
    if plan is not None and q.is_cuda and q.dtype == torch.bfloat16 and k is not None and not score_hook:
        out = attention_fast.decode_fresh(q, k, v, cos, sin, rotary_dim, block_table, k_pool, v_pool, n_heads,
                                          n_kv_heads, head_dim, float(scale), int(window), plan)
        if out is not None:
            return out
    rope_cache_write(q, k, v, cos, sin, rotary_dim, token_seq, token_pos, block_table, k_pool, v_pool,
                     n_heads, n_kv_heads, head_dim, write_cache=k is not None)
    return attention(q, k_pool, v_pool, token_seq, token_pos, block_table, n_heads, n_kv_heads, head_dim,
                     scale, window, plan=plan, score_hook=score_hook)


def qkv_rope_cache(x, w_qkv, cos, sin, rotary_dim, token_seq, token_pos, block_table, k_pool, v_pool,
                   n_heads, n_kv_heads, head_dim):
    """The Q/K/V product of a prompt step with the rotation and the cache write in its epilogue: returns
    the rotated queries [T, nh*hd] (the rotated keys and the values are in the cache), or None when the
    step is not one the tcgen05 product takes this way (few rows, other head sizes, a partial rotation,
    float32) - the caller then runs ``linear`` and ``rope_cache_attention``.  Same bits as those."""
    q_cols, kv_cols = n_heads * head_dim, n_kv_heads * head_dim
    if isinstance(x, ScaledRows) or not x.is_cuda \
            or not gemm_tc.takes_qkv(x, w_qkv, q_cols, kv_cols, head_dim, rotary_dim, cos, sin, k_pool, v_pool):
        return None
    _need_cuda(x, w_qkv, cos, sin, token_seq, token_pos, block_table, k_pool, v_pool)
    _check_pools(k_pool, v_pool, n_kv_heads, head_dim)
    _int32(token_seq, "token_seq")
    _int32(token_pos, "token_pos")
    _int32(block_table, "block_table")
    if token_pos.numel() != x.shape[0] or token_seq.numel() != x.shape[0] or cos.shape != sin.shape \
            or cos.shape[1] != head_dim // 2:
        raise KernelError("qkv_rope_cache: one position and sequence per row, tables [positions, head_dim/2]")
    return gemm_tc.run_qkv(x, w_qkv, q_cols, kv_cols, head_dim, n_kv_heads, cos, sin, token_pos, token_seq, block_table,
                           k_pool, v_pool)


# ---------------------------------------------------------------- feed-forward
def swiglu(gate_up):
    """silu(gate) * up for gate_up = [gate | up] of shape [T, 2I]; returns [T, I]."""
    _need_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelError("swiglu: need a contiguous [T, 2I] tensor")
    rows, two_i = gate_up.shape
    width = two_i // 2
    out = torch.empty((rows, width), dtype=gate_up.dtype, device=gate_up.device)
    esize = gate_up.element_size()
    _library.call("dl_swiglu", gate_up.data_ptr(), gate_up.data_ptr() + width * esize, two_i,
                  _ptr(out), _code(gate_up.dtype), rows, width, _stream())
    return out


# --------------------------------------------------------------------- linear
def linear(x, w, out_dtype=None, resident=False, lazy=False):
    """y = x W^T for W [N, K].  ``resident``: the caller vouches that nothing still pending on the
    stream writes W (a model's weights), which lets the decode kernel start streaming W while
    the kernel before it finishes.  ``lazy`` (float32 results of bfloat16 rows): return a
    PendingProduct, for a caller whose result goes to ``add_rmsnorm`` as the delta.  x may be a
    ScaledRows.

    float32: the library's own FFMA kernel (true 32-bit, the same bits for any number of rows).
    bfloat16: cuBLAS through torch with float32 accumulation, the library product that the
    reference also uses for its projections (src/DotLLM.Cuda/CudaGemm.cs:29-40)."""
    given, rows = x, None
    if isinstance(x, ScaledRows):
        if gemm_skinny.takes(x.data, w):
            rows, x = x.row_sums(), x.data
        else:
            given = x = x.tensor()
    _need_cuda(x, w)
    if w.dim() != 2 or not w.is_contiguous() or x.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KernelError(f"linear: x {tuple(x.shape)} does not match W {tuple(w.shape)}")
    if x.dtype != w.dtype:
        raise KernelError(f"linear: x is {x.dtype} but W is {w.dtype}")
    out_dtype = out_dtype or x.dtype
    M, K = x.shape
    N = w.shape[0]
    if lazy and out_dtype == torch.float32 and x.dtype == torch.bfloat16 and M > 0:
        return PendingProduct(given, w, resident)
    if rows is not None:
        return gemm_skinny.run(x, w, out_dtype, resident=resident, row_sums=rows)
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise KernelError("linear: the float32 product writes float32")
        xs = _rows_view(x, "linear x")
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
        _library.call("dl_gemm_f32", _ptr(x), xs, _ptr(w), _ptr(y), N, M, N, K, _stream())
        return y
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtype {x.dtype}")
    if M > 0:
        y = gemm_skinny.maybe_run(x, w, out_dtype, resident=resident)
        if y is not None:
            return y
    if out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


def gated_linear(x, w_gate_up, resident=False):
    """silu(x Wg^T) * (x Wu^T) for W = [Wg; Wu] of shape [2I, K]; returns [T, I] in x's dtype.
    In bfloat16 one kernel does the product and the gating in float32: the weight-streaming
    kernel for a few rows, the tcgen05 kernel for many.  In float32 the product is followed by
    the gating kernel."""
    if isinstance(x, ScaledRows):
        if w_gate_up.dim() == 2 and x.shape[1] == w_gate_up.shape[1] and gemm_skinny.takes(x.data, w_gate_up, True):
            _need_cuda(x.data, w_gate_up)
            return gemm_skinny.run(x.data, w_gate_up, x.dtype, fuse_swiglu=True, resident=resident, row_sums=x.row_sums())
        x = x.tensor()
    _need_cuda(x, w_gate_up)
    if w_gate_up.dim() != 2 or w_gate_up.shape[0] % 2 or not w_gate_up.is_contiguous() or x.dim() != 2 \
            or x.shape[1] != w_gate_up.shape[1]:
        raise KernelError(f"gated_linear: x {tuple(x.shape)} does not match W {tuple(w_gate_up.shape)}")
    if x.dtype == torch.bfloat16 and x.shape[0] > 0:
        y = gemm_skinny.maybe_run(x, w_gate_up, x.dtype, fuse_swiglu=True, resident=resident)
        if y is not None:
            return y
        if gemm_tc.takes(x, w_gate_up, fuse_swiglu=True):
            return gemm_tc.run(x, w_gate_up, x.dtype, fuse_swiglu=True)
    return swiglu(linear(x, w_gate_up))


# ------------------------------------------------------------------- sampling
def sample(logits, temperature=None, top_k=None, top_p=None, min_p=None, uniform=None, out=None, split=None):
    """One token per row of float32 logits [R, V].  With ``temperature`` None every row is
    greedy (first index of the maximum).  Otherwise per-row float32/int32 tensors [R] give the
    chain temperature -> top-k -> top-p -> min-p and ``uniform`` the draw in [0, 1);
    a row with temperature <= 0 is greedy.  ``split``: None lets the library choose between one
    block per row and a cluster of blocks per row (long rows, few of them); False / True force
    one or the other - they give the same tokens."""
    _need_cuda(logits, temperature, top_k, top_p, min_p, uniform)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 [rows, vocab] with contiguous rows")
    rows, vocab = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                        ("uniform", uniform, torch.float32)):
        if t is not None and (t.dtype != dt or t.shape != (rows,) or not t.is_contiguous()):
            raise KernelError(f"sample: {name} must be a contiguous {dt} tensor of {rows} values")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    elif out.dtype != torch.int32 or out.shape != (rows,) or not out.is_contiguous() or not out.is_cuda:
        raise KernelError("sample: out must be a contiguous int32 CUDA tensor of one id per row")
    _library.call("dl_sample", _ptr(logits), logits.stride(0) if rows > 1 else vocab, rows, vocab,
                  _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform), _ptr(out),
                  0 if split is None else (2 if split else 1), _stream())
    return out


def repetition_penalty(logits, prev, prev_len, penalty, window, row_map=None, append=None):
    """In place: each distinct id among the last ``window[r]`` (0 = all) of row r's
    ``prev[r, :prev_len[r]]`` has its logit divided (if positive) or multiplied by ``penalty[r]``.
    ``row_map`` (int32 [rows]): row r's ids are in ``prev[row_map[r]]`` instead.  ``append`` =
    (positions, ids), int32 [rows] each: before anything else id r is written at ``prev[row, positions[r]]``
    (a position < 0: nothing), for callers that keep the histories on the device and send one id a step."""
    _need_cuda(logits, prev, prev_len, penalty, window, row_map)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("repetition_penalty: logits must be float32 [rows, vocab]")
    rows, vocab = logits.shape
    if prev.dtype != torch.int32 or prev.dim() != 2 or not prev.is_contiguous() or (row_map is None and prev.shape[0] < rows):
        raise KernelError("repetition_penalty: prev must be contiguous int32 [rows, n]")
    _int32(prev_len, "prev_len")
    _int32(window, "window")
    if row_map is not None:
        _int32(row_map, "row_map")
    pos = tok = None
    if append is not None:
        pos, tok = append
        _need_cuda(pos, tok)
        _int32(pos, "append positions")
        _int32(tok, "append ids")
    if penalty.dtype != torch.float32 or not penalty.is_contiguous():
        raise KernelError("repetition_penalty: penalty must be float32 [rows]")
    for name, t in (("prev_len", prev_len), ("window", window), ("penalty", penalty), ("row_map", row_map), ("append positions", pos),
                    ("append ids", tok)):
        if t is not None and t.numel() != rows:
            raise KernelError(f"repetition_penalty: {name} must hold one value per row ({rows}), got {t.numel()}")
    _library.call("dl_repetition_penalty", _ptr(logits), logits.stride(0) if rows > 1 else vocab, rows,
                  vocab, _ptr(prev), prev.shape[1], prev.shape[0], _ptr(row_map), _ptr(pos), _ptr(tok), _ptr(prev_len),
                  _ptr(penalty), _ptr(window), _stream())
    return logits
