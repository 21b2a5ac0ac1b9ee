"""Python entry points of the routed feed-forward (csrc/routed_experts.cu)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, check, core, dtype_code, need_contiguous, ptr, stream, tc_status_word


def table_choice(tokens: torch.Tensor, table: torch.Tensor, n_experts: int) -> torch.Tensor:
    """choice[t, s] = table[tokens[t], s]: the experts of each token of the step (int32 [T, top])."""
    if tokens.dtype != torch.int32 or table.dtype != torch.int32 or table.dim() != 2:
        raise KernelError("table_choice: tokens int32 [T], table int32 [vocab, top]")
    need_contiguous(tokens=tokens, table=table)
    T, (vocab, top) = tokens.shape[0], table.shape
    choice = torch.empty((T, top), dtype=torch.int32, device=tokens.device)
    check(core().tq_table_choice(ptr(tokens), ptr(table), vocab, top, n_experts, ptr(choice), T, stream()),
          "table_choice")
    return choice


def router_choice(logits: torch.Tensor, top: int, scale: float, floor: float) -> tuple[torch.Tensor, torch.Tensor]:
    """From a router's float32 logits [T, E]: the `top` experts with the largest sigmoid(logit) per token
    (int32 [T, top], the lowest index first among equals) and their weights scale * s / (sum of the chosen s +
    floor) (float32 [T, top])."""
    T, E = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or not 1 <= top <= E:
        raise KernelError("router_choice: float32 logits [T, E], 1 <= top <= E")
    choice = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    check(core().tq_router_choice(ptr(logits), logits.stride(0), E, top, float(scale), float(floor), ptr(choice),
                                  ptr(weights), T, stream()), "router_choice")
    return choice, weights


def _check_weights(weights, choice):
    if weights is not None and (weights.dtype != torch.float32 or weights.shape != choice.shape
                                or not weights.is_contiguous()):
        raise KernelError("routed_experts: weights float32 of choice's shape")


def routed_experts_rows(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, choice: torch.Tensor,
                        y: torch.Tensor, accumulate: bool, weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y (=, +=) mean over a token's experts e (with `weights` float32 [T, top]: the sum weighted by them) of
    w_down[e] (silu(gate[e] x) * (up[e] x)), every (token, expert)
    pair a row-times-matrix product of its own.  x [T, W]; w_gate_up [E, 2F, W]; w_down [E, W, F];
    choice int32 [T, top]; y float32 [T, W]."""
    T, W = x.shape
    E, F2, W2 = w_gate_up.shape
    F = F2 // 2
    if W2 != W or tuple(w_down.shape) != (E, W, F) or w_down.dtype != w_gate_up.dtype:
        raise KernelError(f"routed_experts: weights {tuple(w_gate_up.shape)} / {tuple(w_down.shape)} do not fit width {W}")
    if choice.dtype != torch.int32 or choice.shape[0] != T or y.dtype != torch.float32 or tuple(y.shape) != (T, W):
        raise KernelError("routed_experts: choice int32 [T, top], y float32 [T, W]")
    if x.stride(1) != 1:
        raise KernelError("routed_experts: x must be contiguous along its rows")
    need_contiguous(w_gate_up=w_gate_up, w_down=w_down, choice=choice, y=y)
    _check_weights(weights, choice)
    top = choice.shape[1]
    act = torch.empty((T * top, F), dtype=x.dtype, device=x.device)
    check(core().tq_routed_experts_rows(ptr(x), dtype_code(x), x.stride(0), ptr(w_gate_up), ptr(w_down),
                                        dtype_code(w_down), ptr(choice), ptr(weights), top, T, W, F, ptr(act), ptr(y),
                                        int(accumulate), stream()), "routed_experts_rows", 2)
    return y


TILE_ROWS = 128                     # rows of a tile of the tensor-core products (csrc/gemm_tc.cu)


def routed_tiles_ok(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    """Whether the sorted-tiles form takes these operands: bfloat16 throughout, rows of whole 16-byte pieces."""
    E, F2, W = w_gate_up.shape
    F = F2 // 2
    return (x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
            and W % 8 == 0 and F % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)


def routed_experts_tiles(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, choice: torch.Tensor,
                         y: torch.Tensor, accumulate: bool, weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same result as `routed_experts_rows` for many rows: the (token, expert) pairs are sorted by expert
    into a buffer in which every expert owns whole tiles of 128 rows; two tensor-core products over the whole
    buffer follow, in which each tile multiplies with its own expert's matrices (the first gates, silu(g) * u,
    in its epilogue), and a last kernel takes each token's rows back and averages them."""
    T, W = x.shape
    E, F2, _ = w_gate_up.shape
    F = F2 // 2
    if not routed_tiles_ok(x, w_gate_up, w_down) or tuple(w_down.shape) != (E, W, F):
        raise KernelError("routed_experts_tiles: bfloat16 operands with widths in multiples of 8")
    if choice.dtype != torch.int32 or choice.shape[0] != T or y.dtype != torch.float32 or tuple(y.shape) != (T, W):
        raise KernelError("routed_experts: choice int32 [T, top], y float32 [T, W]")
    need_contiguous(w_gate_up=w_gate_up, w_down=w_down, choice=choice, y=y)
    _check_weights(weights, choice)
    top = choice.shape[1]
    n_pairs = T * top
    max_tiles = n_pairs // TILE_ROWS + E
    rows = max_tiles * TILE_ROWS
    dev = x.device
    plan = torch.empty(n_pairs + 2 * max_tiles, dtype=torch.int32, device=dev)
    pos, tile_up, tile_down = plan[:n_pairs], plan[n_pairs:n_pairs + max_tiles], plan[n_pairs + max_tiles:]
    sorted_x = torch.empty((rows, W), dtype=torch.bfloat16, device=dev)
    act = torch.empty((rows, F), dtype=torch.bfloat16, device=dev)
    out = torch.empty((rows, W), dtype=torch.float32, device=dev)
    lib = core()
    check(lib.tq_routed_sort(ptr(x), x.stride(0), ptr(choice), top, T, W, E, TILE_ROWS, 2 * F, W, max_tiles, ptr(pos),
                             ptr(tile_up), ptr(tile_down), ptr(sorted_x), stream()), "routed_sort", 2)
    status = ptr(tc_status_word(dev))
    check(lib.tq_gemm_tc_grouped(ptr(sorted_x), ptr(w_gate_up), ptr(act), dtype_code(act), rows, F, W, W, W, F,
                                 2, E * 2 * F, F, ptr(tile_up), status, stream()), "routed_gate_up")
    check(lib.tq_gemm_tc_grouped(ptr(act), ptr(w_down), ptr(out), dtype_code(out), rows, W, F, F, F, W,
                                 0, E * W, 0, ptr(tile_down), status, stream()), "routed_down")
    check(lib.tq_routed_combine(ptr(out), ptr(pos), ptr(weights), top, T, W, ptr(y), int(accumulate), stream()),
          "routed_combine")
    return y
