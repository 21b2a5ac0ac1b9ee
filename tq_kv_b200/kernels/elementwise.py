"""Python entry points of the memory-bound kernels (csrc/elementwise.cu)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, check, core, dtype_code, need_contiguous, ptr, stream


def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None,
          scale: float = 1.0):
    """out[t] = scale * float32(table[tokens[t]]).  tokens int32 [T]; table [V, H]
    float32 or bfloat16; out float32 [T, H].  `status` (int32 [1]) gets bit 0
    set if a token id lies outside the table."""
    T = tokens.shape[0]
    V, H = table.shape
    if tokens.dtype != torch.int32 or out.dtype != torch.float32 or tuple(out.shape) != (T, H):
        raise KernelError("embed: tokens must be int32 [T] and out float32 [T, H]")
    need_contiguous(tokens=tokens, table=table, out=out)
    check(core().tq_embed_scaled(ptr(tokens), ptr(table), dtype_code(table), ptr(out), T, H, V, ptr(status),
                                 float(scale), stream()), "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None):
    """out[r] = x[rows[r] or r] / sqrt(mean(x^2) + eps) * weight.  x float32
    [*, H]; weight float32 [H]; out float32 or bfloat16 [R, H]."""
    H = x.shape[-1]
    R = out.shape[0]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or weight.shape[0] != H or out.shape[-1] != H:
        raise KernelError("rmsnorm: x and weight must be float32 with matching width")
    if rows is None and x.shape[0] != R:
        raise KernelError("rmsnorm: out must have as many rows as x when no rows are selected")
    if rows is not None and (rows.dtype != torch.int32 or rows.shape[0] != R):
        raise KernelError("rmsnorm: rows must be int32 [R]")
    need_contiguous(x=x, weight=weight, out=out, rows=rows)
    check(core().tq_rmsnorm(ptr(x), ptr(weight), ptr(out), dtype_code(out), ptr(rows), R, H, float(eps), stream()),
          "rmsnorm")
    return out


def qkv_rope_cache(qkv, bias, cos, sin, tok_pos, tok_seq, new_lens, q_out, *, n_heads, n_kv_heads, head_dim,
                   rotary_dim, k_out=None, v_out=None, k_pages=None, v_pages=None, block_table=None,
                   table_width=0, ring_pages=0, page_tokens=64, clear_input=False):
    """Bias, rotary encoding of q and k, head split, cache append (see
    csrc/elementwise.cu).  qkv [T, (nh+2nkv)*hd]; cos/sin float32
    [positions, rotary_dim/2]; q_out/k_out/v_out and the pages share one dtype.
    With `clear_input` the kernel leaves zeros in the rows of qkv it has read."""
    T = qkv.shape[0]
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"qkv_rope_cache: qkv has width {qkv.shape[1]}, expected {width}")
    if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
        raise KernelError(f"qkv_rope_cache: rotary_dim {rotary_dim} must be even and within head_dim {head_dim}")
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape[1] != rotary_dim // 2:
        raise KernelError("qkv_rope_cache: cos/sin must be float32 [positions, rotary_dim/2]")
    for t in (k_out, v_out, k_pages, v_pages):
        if t is not None and t.dtype != q_out.dtype:
            raise KernelError("qkv_rope_cache: outputs and cache pages must share one dtype")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape[0] != width):
        raise KernelError("qkv_rope_cache: bias must be float32 of the qkv width")
    need_contiguous(qkv=qkv, bias=bias, cos=cos, sin=sin, q_out=q_out, k_out=k_out, v_out=v_out, k_pages=k_pages,
                    v_pages=v_pages)
    check(core().tq_qkv_rope_cache(
        ptr(qkv), dtype_code(qkv), ptr(bias), ptr(cos), ptr(sin), ptr(tok_pos), ptr(tok_seq), ptr(new_lens),
        ptr(block_table), table_width, ring_pages, page_tokens, ptr(q_out), ptr(k_out), ptr(v_out), ptr(k_pages),
        ptr(v_pages), dtype_code(q_out), T, n_heads, n_kv_heads, head_dim, rotary_dim, int(clear_input), stream()),
        "qkv_rope_cache")


ACT_SILU, ACT_GELU_TANH = 1, 2          # the gate's activation in a gated feed-forward (csrc/common.cuh)


def activation_code(name: str) -> int:
    try:
        return {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH}[name]
    except KeyError:
        raise KernelError(f"unknown gate activation '{name}' (silu, gelu_tanh)") from None


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, act: int = ACT_SILU):
    """out = act(gate) * up for gate_up [T, 2I] = [gate | up]; act: silu (the default) or the tanh form of gelu."""
    T, I2 = gate_up.shape
    I = I2 // 2
    if I2 % 2 or tuple(out.shape) != (T, I):
        raise KernelError("swiglu: gate_up must be [T, 2I] and out [T, I]")
    need_contiguous(gate_up=gate_up, out=out)
    check(core().tq_swiglu(ptr(gate_up), dtype_code(gate_up), ptr(out), dtype_code(out), T, I, int(act), stream()),
          "swiglu")
    return out


def add_into(acc: torch.Tensor, x: torch.Tensor):
    """acc += float32(x), acc float32."""
    if acc.dtype != torch.float32 or acc.shape != x.shape:
        raise KernelError("add_into: acc must be float32 and of x's shape")
    need_contiguous(acc=acc, x=x)
    check(core().tq_add_into(ptr(acc), ptr(x), dtype_code(x), acc.numel(), stream()), "add_into")
    return acc


def select_tokens(tokens: torch.Tensor, source_rows: torch.Tensor, sampled: torch.Tensor):
    """tokens[i] = sampled[source_rows[i]] where source_rows[i] >= 0; other
    entries keep the id the host put there.  All int32, on the device: the
    token a sequence decodes next can be the one the sampler just chose,
    without a trip through the host."""
    n = tokens.shape[0]
    for name, t in (("tokens", tokens), ("source_rows", source_rows), ("sampled", sampled)):
        if t.dtype != torch.int32:
            raise KernelError(f"select_tokens: {name} must be int32")
    if source_rows.shape[0] < n:
        raise KernelError("select_tokens: one source row per token")
    need_contiguous(tokens=tokens, source_rows=source_rows, sampled=sampled)
    check(core().tq_select_tokens(ptr(tokens), ptr(source_rows), ptr(sampled), n, stream()), "select_tokens")
    return tokens


def random_fill(out: torch.Tensor, key: int, std: float, offset: float = 0.0):
    """out[i] = offset + std * z(key, i) with z standard normal from the
    counter-based generator of csrc/random_fill.cu (float32 or bfloat16 out)."""
    need_contiguous(out=out)
    check(core().tq_random_fill(ptr(out), dtype_code(out), out.numel(), int(key) & ((1 << 64) - 1), float(std),
                                float(offset), stream()), "random_fill")
    return out


def embed_sinusoid(tokens: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, rate: torch.Tensor,
                   out: torch.Tensor, status: Optional[torch.Tensor] = None):
    """out[t, c] = float32(table[tokens[t], c]) + (sin if c is even else cos)(positions[t] * rate[c // 2]).
    tokens, positions int32 [T]; rate float32 [ceil(H / 2)]; out float32 [T, H]."""
    T = tokens.shape[0]
    V, H = table.shape
    if tokens.dtype != torch.int32 or positions.dtype != torch.int32 or positions.shape[0] < T:
        raise KernelError("embed_sinusoid: tokens and positions must be int32 [T]")
    if out.dtype != torch.float32 or tuple(out.shape) != (T, H):
        raise KernelError("embed_sinusoid: out must be float32 [T, H]")
    if rate.dtype != torch.float32 or rate.shape[0] < (H + 1) // 2:
        raise KernelError("embed_sinusoid: rate must be float32 [ceil(H / 2)]")
    need_contiguous(tokens=tokens, positions=positions, table=table, rate=rate, out=out)
    check(core().tq_embed_sinusoid(ptr(tokens), ptr(positions), ptr(table), dtype_code(table), ptr(rate), ptr(out), T, H,
                                   V, ptr(status), stream()), "embed_sinusoid")
    return out


GATE_SIGMOID, GATE_SILU, GATE_SILU_FIRST = 0, 1, 2


def group_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *, groups: int = 1,
                  gate: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                  gate_mode: int = GATE_SIGMOID):
    """RMS norm in `groups` consecutive groups of a row, times `weight`, optionally times sigmoid(gate) entry by
    entry (`gate_mode` GATE_SILU: times silu(gate) instead; GATE_SILU_FIRST: x times silu(gate) BEFORE the norm).  x float32 [*, W] and gate float32 [*, W] may be column slices of wider buffers (row strides are
    passed on); weight float32 [W]; out float32 or bfloat16 [R, W]."""
    W = x.shape[-1]
    R = out.shape[0]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or weight.shape[0] != W or out.shape[-1] != W:
        raise KernelError("group_rmsnorm: x and weight must be float32 with matching width")
    if groups < 1 or W % groups:
        raise KernelError(f"group_rmsnorm: a width of {W} cannot be cut into {groups} equal groups")
    if x.stride(-1) != 1 or out.stride(-1) != 1 or (gate is not None and (gate.stride(-1) != 1 or gate.dtype != torch.float32
                                                                        or gate.shape != x.shape)):
        raise KernelError("group_rmsnorm: x, gate and out must be contiguous along the row; gate float32 of x's shape")
    if rows is None and x.shape[0] != R:
        raise KernelError("group_rmsnorm: out must have as many rows as x when no rows are selected")
    if rows is not None and (rows.dtype != torch.int32 or rows.shape[0] != R):
        raise KernelError("group_rmsnorm: rows must be int32 [R]")
    need_contiguous(weight=weight, rows=rows)
    check(core().tq_group_rmsnorm(ptr(x), x.stride(0), ptr(weight), ptr(gate), 0 if gate is None else gate.stride(0),
                                  ptr(out), dtype_code(out), out.stride(0), ptr(rows), R, W, groups, float(eps),
                                  int(gate_mode), stream()), "group_rmsnorm")
    return out


def add_normed(acc: torch.Tensor, sources, eps: float, scale: float):
    """acc[t] += scale * sum over (x, w) in sources of x[t] / sqrt(mean(x[t]^2) + eps) * w.  acc and every x
    float32 [T, W] contiguous, every w float32 [W]; up to four sources."""
    T, W = acc.shape
    sources = list(sources)
    if not 1 <= len(sources) <= 4:
        raise KernelError("add_normed: one to four sources")
    flat = []
    for x, w in sources:
        if x.dtype != torch.float32 or w.dtype != torch.float32 or tuple(x.shape) != (T, W) or w.shape[0] != W:
            raise KernelError("add_normed: sources must be float32 [T, W] with float32 weights [W]")
        need_contiguous(x=x, w=w)
        flat += [ptr(x), ptr(w)]
    flat += [None] * (8 - len(flat))
    if acc.dtype != torch.float32:
        raise KernelError("add_normed: acc must be float32")
    need_contiguous(acc=acc)
    check(core().tq_add_normed(ptr(acc), *flat, len(sources), T, W, float(eps), float(scale), stream()), "add_normed")
    return acc


def add_scaled(acc: torch.Tensor, x: torch.Tensor, scale: float):
    """acc += scale * x, both float32 and contiguous."""
    if acc.dtype != torch.float32 or x.dtype != torch.float32 or acc.shape != x.shape:
        raise KernelError("add_scaled: acc and x must be float32 of one shape")
    need_contiguous(acc=acc, x=x)
    check(core().tq_add_scaled(ptr(acc), ptr(x), acc.numel(), float(scale), stream()), "add_scaled")
    return acc


def tanh_rows(x: torch.Tensor, out: torch.Tensor):
    """out = tanh(x) for float32 x [T, n] (may be a column slice: its row stride is passed on)."""
    T, n = x.shape
    if x.dtype != torch.float32 or tuple(out.shape) != (T, n) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("tanh_rows: x float32 [T, n], out [T, n], both contiguous along the row")
    check(core().tq_tanh_rows(ptr(x), x.stride(0), ptr(out), dtype_code(out), out.stride(0), T, n, stream()), "tanh_rows")
    return out


def scale_inplace(x: torch.Tensor, s: float):
    """x *= s for a contiguous float32 tensor."""
    if x.dtype != torch.float32:
        raise KernelError("scale_inplace: x must be float32")
    need_contiguous(x=x)
    check(core().tq_scale_inplace(ptr(x), x.numel(), float(s), stream()), "scale_inplace")
    return x


def head_encode(proj: torch.Tensor, ctx_pos, q_out: torch.Tensor, *, q_col: int, k_col: int, v_col: int,
                n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, cos=None, sin=None, rotary_dim: int = 0,
                norm_eps: float = 0.0, k_out=None, v_out=None, k_pages=None, v_pages=None, block_table=None,
                table_width: int = 0, ring_pages: int = 0, page_tokens: int = 64, paired: bool = False,
                row_inv=None, q_weight=None, k_weight=None):
    """From projected float32 rows [T, ld] (q heads from column q_col, k heads from k_col, v heads from v_col; with
    v_col < 0 the values are the keys as projected) to encoded q, and k / v packed and / or appended to the cache
    (see csrc/head_encode.cu).  `ctx_pos` = (tok_pos, tok_seq, new_lens).  q and k are rotated over their first
    `rotary_dim` entries (cos/sin float32 [positions, rotary_dim/2]; entry i with i + rotary_dim/2, or with
    `paired` entry 2i with 2i + 1) or, with norm_eps > 0, divided by their root mean square per head.  With
    `row_inv` (float32 [T, 2] from `row_inv_rms`) and the weights q_weight [n_heads * key_dim] and k_weight
    [n_kv_heads * key_dim], q and k are first normed over their whole rows.  n_kv_heads may be 0: only q is encoded."""
    tok_pos, tok_seq, new_lens = ctx_pos
    T, ld = proj.shape
    if proj.dtype != torch.float32 or proj.stride(1) != 1:
        raise KernelError("head_encode: the projected rows must be float32")
    if rotary_dim:
        if rotary_dim % 2 or rotary_dim > key_dim or cos is None or cos.dtype != torch.float32 \
                or cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"head_encode: rotary_dim {rotary_dim} needs float32 tables [positions, {rotary_dim // 2}]")
    if n_kv_heads and v_col < 0 and value_dim != key_dim:
        raise KernelError("head_encode: values that are the keys have the keys' width")
    need = max(q_col + n_heads * key_dim, k_col + n_kv_heads * key_dim, v_col + n_kv_heads * value_dim if v_col >= 0 else 0)
    if need > ld or min(q_col, k_col) < 0:
        raise KernelError(f"head_encode: the columns reach {need}, the rows have {ld}")
    for t in (k_out, v_out, k_pages, v_pages):
        if t is not None and t.dtype != q_out.dtype:
            raise KernelError("head_encode: all outputs and the cache must share one dtype")
    if row_inv is not None:
        if (row_inv.dtype != torch.float32 or tuple(row_inv.shape) != (T, 2) or q_weight is None
                or q_weight.dtype != torch.float32 or q_weight.shape[0] != n_heads * key_dim
                or (n_kv_heads and (k_weight is None or k_weight.dtype != torch.float32
                                    or k_weight.shape[0] != n_kv_heads * key_dim))):
            raise KernelError("head_encode: row_inv float32 [T, 2] needs float32 weights over the whole q and k rows")
        need_contiguous(row_inv=row_inv, q_weight=q_weight, k_weight=k_weight)
    need_contiguous(q_out=q_out, k_out=k_out, v_out=v_out, k_pages=k_pages, v_pages=v_pages, block_table=block_table,
                    cos=cos, sin=sin)
    check(core().tq_head_encode(ptr(proj), proj.stride(0), q_col, k_col, v_col, ptr(cos), ptr(sin), rotary_dim,
                                float(norm_eps), ptr(tok_pos), ptr(tok_seq), ptr(new_lens), ptr(block_table),
                                table_width, ring_pages, page_tokens, ptr(q_out), ptr(k_out), ptr(v_out), ptr(k_pages),
                                ptr(v_pages), dtype_code(q_out), T, n_heads, n_kv_heads, key_dim, value_dim,
                                ptr(row_inv), ptr(q_weight), ptr(k_weight), int(bool(paired)), stream()),
          "head_encode")
    return q_out


def row_inv_rms(proj: torch.Tensor, *, q_col: int, q_width: int, q_count: int, k_col: int = 0, k_width: int = 0,
                k_count: int = 0, eps: float) -> torch.Tensor:
    """float32 [T, 2]: per token 1 / sqrt(sum(q row^2) / q_count + eps) over columns q_col .. q_col + q_width of
    the float32 rows `proj`, and the same for the k row (k_width 0: there is none).  The counts are the rows' true
    lengths where they are padded with zeros."""
    T, ld = proj.shape
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or q_col + q_width > ld or k_col + k_width > ld:
        raise KernelError("row_inv_rms: float32 rows that hold both projections")
    out = torch.empty((T, 2), dtype=torch.float32, device=proj.device)
    check(core().tq_row_inv_rms(ptr(proj), proj.stride(0), q_col, q_width, q_count, k_col, k_width, k_count,
                                float(eps), ptr(out), T, stream()), "row_inv_rms")
    return out


def add_normed_copy(acc: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                    copy: Optional[torch.Tensor] = None):
    """acc[t] += y[t] / sqrt(mean(y[t]^2) + eps) * weight, and `copy` (bfloat16 or float32 [T, W], if given)
    receives the new acc rounded to its type.  acc, y float32 [T, W] contiguous; weight float32 [W]."""
    T, W = acc.shape
    if acc.dtype != torch.float32 or y.dtype != torch.float32 or tuple(y.shape) != (T, W) \
            or weight.dtype != torch.float32 or weight.shape[0] != W:
        raise KernelError("add_normed_copy: acc and y float32 [T, W], weight float32 [W]")
    if copy is not None and tuple(copy.shape) != (T, W):
        raise KernelError("add_normed_copy: the copy must be [T, W]")
    need_contiguous(acc=acc, y=y, weight=weight, copy=copy)
    check(core().tq_add_normed_copy(ptr(acc), ptr(y), ptr(weight), T, W, float(eps), ptr(copy),
                                    0 if copy is None else dtype_code(copy), stream()), "add_normed_copy")
    return acc


def round_rows(x: torch.Tensor) -> torch.Tensor:
    """The float32 tensor x rounded to bfloat16."""
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("round_rows: x must be contiguous float32")
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    check(core().tq_round_rows(ptr(x), ptr(out), x.numel(), stream()), "round_rows")
    return out


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor):
    """x[t, i] *= sigmoid(gate[t, i]) in place; gate float32, possibly a column slice of wider rows."""
    T, n = x.shape
    if gate.dtype != torch.float32 or tuple(gate.shape) != (T, n) or gate.stride(1) != 1 or not x.is_contiguous():
        raise KernelError("sigmoid_gate: gate must be float32 of x's shape, x contiguous")
    check(core().tq_sigmoid_gate(ptr(x), dtype_code(x), ptr(gate), gate.stride(0), T, n, stream()), "sigmoid_gate")
    return x


def tanh_cap(x: torch.Tensor, cap: float):
    """x <- cap * tanh(x / cap) in place (float32)."""
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("tanh_cap: x must be contiguous float32")
    check(core().tq_tanh_cap(ptr(x), x.numel(), float(cap), stream()), "tanh_cap")
    return x
