"""Expert-parallel MoE: routing plan, fp8 dispatch, grouped expert FFN, weighted combine
(csrc/kernels/moe.cu).  Everything stays on the device: token counts per expert are exchanged with
this library's all-gather and turned into receive offsets with a few tensor ops, and the grouped
GEMM reads the per-expert row ranges from device memory, so no step needs the host to know sizes.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .._native import C
from ..engine import Engine
from . import collectives as coll
from .gemm import count_launch, status_words


def quant_fp8_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, hidden] -> (e4m3 bytes [rows, hidden], fp32 scales [rows, hidden/128]); 1 x 128 blocks."""
    rows, hidden = x.shape
    q = torch.empty((rows, hidden), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, hidden // 128), dtype=torch.float32, device=x.device)
    C.quant_fp8_rows(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, hidden, torch.cuda.current_stream().cuda_stream)
    count_launch()
    return q, s


def quant_fp8_blocks(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [rows, cols] weights -> (e4m3 bytes, fp32 scales [rows/128, cols/128]); 128 x 128 blocks."""
    rows, cols = w.shape
    q = torch.empty((rows, cols), dtype=torch.uint8, device=w.device)
    s = torch.empty((rows // 128, cols // 128), dtype=torch.float32, device=w.device)
    C.quant_fp8_blocks(w.data_ptr(), q.data_ptr(), s.data_ptr(), rows, cols, torch.cuda.current_stream().cuda_stream)
    count_launch()
    return q, s


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, row_off: torch.Tensor, n: int, out: Optional[torch.Tensor] = None,
                 gelu: bool = False) -> torch.Tensor:
    """Rows [row_off[g], row_off[g+1]) of ``a`` [*, K] times ``b[g*n:(g+1)*n]`` ([groups*n, K]) ^T -> same rows of out [*, n]."""
    groups = row_off.numel() - 1
    if out is None:
        out = torch.empty((a.shape[0], n), dtype=torch.bfloat16, device=a.device)
    C.gemm_grouped(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0), row_off.data_ptr(), groups,
                   a.shape[0], n, a.shape[1], C.GEMM_GELU_INPLACE if gelu else 0, 0, status_words().data_ptr(),
                   torch.cuda.current_stream().cuda_stream)
    count_launch()
    return out


class MoEExchange:
    """Buffers and kernels of one expert-parallel MoE layer shape."""

    def __init__(self, eng: Engine, tokens: int, hidden: int, n_experts: int, topk: int, capacity_factor: float = 2.0,
                 blocks: Optional[int] = None, flag_lane: int = 5):
        if n_experts % eng.world or hidden % 128 or topk > 8:
            raise ValueError("MoEExchange: experts must divide over ranks, hidden % 128 == 0, top-k <= 8")
        self.eng, self.T, self.H, self.E, self.K = eng, tokens, hidden, n_experts, topk
        self.epr = n_experts // eng.world
        self.cap = int(capacity_factor * tokens * topk) // 128 * 128 + 128
        self.recv_q = eng.symmetric_tensor((self.cap, hidden), torch.uint8)
        self.recv_s = eng.symmetric_tensor((self.cap, hidden // 128), torch.float32)
        self.y = eng.symmetric_tensor((self.cap, hidden), torch.bfloat16)
        self.counts_all = eng.symmetric_tensor((eng.world, n_experts), torch.int32)
        self.x_bf16 = torch.empty((self.cap, hidden), dtype=torch.bfloat16, device="cuda")
        # de-duplicated exchange: where a row's payload is (alias), the rows and gate weights of a token's group on this
        # rank (64 bytes per row), and the groups' weighted sums of expert outputs
        self.alias = eng.symmetric_tensor((self.cap,), torch.int32)
        self.groups = eng.symmetric_tensor((self.cap, 16), torch.int32)
        self.z = eng.symmetric_tensor((self.cap, hidden), torch.bfloat16)
        self.alias.copy_(torch.arange(self.cap, dtype=torch.int32, device="cuda"))
        self.epoch = 0
        self.blocks = blocks or min(C.sm_count(), C.MAX_BLOCKS_PER_COLL)
        self.flag_lane = flag_lane

    # ---- routing -----------------------------------------------------------------------------
    @staticmethod
    def route(gate_logits: torch.Tensor, topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
        probs = torch.softmax(gate_logits.float(), dim=-1)
        p, ids = probs.topk(topk, dim=-1)
        return ids.to(torch.int32), p.contiguous()

    def plan(self, ids: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Where every (token, k) assignment lands: its row in the destination rank's receive buffer."""
        eng, E, epr = self.eng, self.E, self.epr
        flat = ids.reshape(-1).long()
        counts = torch.bincount(flat, minlength=E).to(torch.int32)
        if eng.world > 1:
            coll.all_gather(eng, counts, self.counts_all.view(-1), lane=self.flag_lane)
            counts_all = self.counts_all
        else:
            counts_all = counts.view(1, E)
        ca = counts_all.long()
        per_expert = ca.sum(0)                                     # rows each expert receives
        grp = per_expert.view(eng.world, epr)
        expert_base = (grp.cumsum(1) - grp).reshape(-1)            # start of the expert's segment on its rank
        src_prefix = (ca.cumsum(0) - ca)[eng.rank]                 # rows of lower ranks inside that segment
        order = torch.argsort(flat, stable=True)
        starts = counts.long().cumsum(0) - counts.long()
        pos_sorted = torch.arange(flat.numel(), device=flat.device) - starts[flat[order]]
        pos = torch.empty_like(pos_sorted)
        pos[order] = pos_sorted
        rows = expert_base[flat] + src_prefix[flat] + pos
        rows = torch.where(rows < self.cap, rows, torch.full_like(rows, -1)).to(torch.int32).view_as(ids)
        mine = grp[eng.rank]
        row_off = torch.zeros(epr + 1, dtype=torch.int32, device=ids.device)
        row_off[1:] = mine.cumsum(0).clamp(max=self.cap).to(torch.int32)
        return {"rows": rows.contiguous(), "row_off": row_off, "n_rows": row_off[-1:].contiguous()}

    def route_and_plan(self, gate_logits: torch.Tensor):
        """Fused routing: one kernel does softmax + top-k + per-expert counting (an assignment's position inside
        its expert's segment is the value its atomic increment returned), the counts are all-gathered, and a
        second kernel turns counts into receive rows.  Returns (ids, probs, plan)."""
        eng, T, K, E = self.eng, self.T, self.K, self.E
        dev = gate_logits.device
        lg = gate_logits.float().contiguous()
        ids = torch.empty((T, K), dtype=torch.int32, device=dev)
        probs = torch.empty((T, K), dtype=torch.float32, device=dev)
        pos = torch.empty((T, K), dtype=torch.int32, device=dev)
        counts = torch.zeros(E, dtype=torch.int32, device=dev)
        s = torch.cuda.current_stream().cuda_stream
        C.moe_route(lg.data_ptr(), ids.data_ptr(), probs.data_ptr(), pos.data_ptr(), counts.data_ptr(), T, E, K, s)
        if eng.world > 1:
            coll.all_gather(eng, counts, self.counts_all.view(-1), lane=self.flag_lane)
            counts_all = self.counts_all
        else:
            counts_all = counts
        rows = torch.empty((T, K), dtype=torch.int32, device=dev)
        row_off = torch.empty(self.epr + 1, dtype=torch.int32, device=dev)
        C.moe_plan(counts_all.data_ptr(), ids.data_ptr(), pos.data_ptr(), rows.data_ptr(), row_off.data_ptr(), eng.world, eng.rank, E,
                   T, K, self.cap, s)
        count_launch(2)
        return ids, probs, {"rows": rows, "row_off": row_off, "n_rows": row_off[-1:]}

    # ---- kernels ----------------------------------------------------------------------------
    def _exchange(self, kind: str, x, ids, rows, probs, out, gate=None, dedupe: bool = False) -> None:
        self.epoch += 1
        st = status_words()
        off = self.eng.heap_offset
        C.moe_exchange(kind, self.eng.raw, [], 0, self.T, self.H, self.K, self.epr, off(self.recv_q),
                       off(self.recv_s), off(self.y), self.epoch, self.flag_lane,
                       [x.data_ptr()] if x is not None else [], [ids.data_ptr()], [rows.data_ptr()],
                       [probs.data_ptr()] if probs is not None else [], [out.data_ptr()] if out is not None else [],
                       [st.data_ptr()], self.blocks, 0, torch.cuda.current_stream().cuda_stream,
                       alias_off=off(self.alias), group_off=off(self.groups), z_off=off(self.z),
                       gate=[gate.data_ptr()] if gate is not None else [], dedupe=dedupe)
        count_launch()

    def dispatch(self, x: torch.Tensor, ids: torch.Tensor, plan: Dict[str, torch.Tensor], probs: Optional[torch.Tensor] = None,
                 gate: Optional[torch.Tensor] = None) -> None:
        """Rows of ``x`` go to the ranks of their experts (e4m3 + block scales).  With ``probs`` destination k of token t
        receives ``probs[t, k] * x[t]`` (how the backward pass sends gate-weighted output gradients).

        With ``gate`` (the routing probabilities; not together with ``probs``) a token crosses NVLink once per destination
        RANK instead of once per expert: the first of its assignments to a rank carries the row, the others are told
        where it is (``received`` / ``experts`` copy it locally while they convert to bf16), and the rank gets the list of
        the token's rows with their gate weights, which ``combine(..., grouped=True)`` needs."""
        if gate is not None and probs is not None:
            raise ValueError("MoEExchange.dispatch: gate (de-duplicated rows) and probs (scaled rows) exclude one another")
        if gate is not None and (gate.dtype != torch.float32 or gate.shape != ids.shape or not gate.is_contiguous()):
            raise ValueError("MoEExchange.dispatch: gate must be a contiguous fp32 [tokens, topk] tensor")
        self._exchange("dispatch", x, ids, plan["rows"], probs, None, gate=gate, dedupe=gate is not None)

    def received(self, plan: Dict[str, torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The rows that the last dispatch delivered to this rank, as bf16 [cap, hidden] (rows past the plan's count are
        not written)."""
        if out is None:
            out = torch.empty((self.cap, self.H), dtype=torch.bfloat16, device="cuda")
        C.moe_dequant(self.recv_q.data_ptr(), self.recv_s.data_ptr(), out.data_ptr(), plan["n_rows"].data_ptr(), self.cap,
                      self.H, torch.cuda.current_stream().cuda_stream, alias=self.alias.data_ptr())
        count_launch()
        return out

    def combine_dot(self, g: torch.Tensor, ids: torch.Tensor, plan: Dict[str, torch.Tensor]) -> torch.Tensor:
        """``dot[t, k] = <g[t], y row of assignment (t, k)>`` (fp32 [tokens, topk]): with ``g`` the upstream gradient and
        the expert outputs of the forward pass still in ``self.y``, the gradient of the gate weights."""
        out = torch.zeros((self.T, self.K), dtype=torch.float32, device="cuda")
        self._exchange("combine_dot", g, ids, plan["rows"], None, out)
        return out

    def experts(self, w1: torch.Tensor, w2: torch.Tensor, plan: Dict[str, torch.Tensor]) -> None:
        """w1: [experts_per_rank * d_ff, hidden], w2: [experts_per_rank * hidden, d_ff]; result in self.y."""
        C.moe_dequant(self.recv_q.data_ptr(), self.recv_s.data_ptr(), self.x_bf16.data_ptr(), plan["n_rows"].data_ptr(), self.cap,
                      self.H, torch.cuda.current_stream().cuda_stream, alias=self.alias.data_ptr())
        count_launch()
        d_ff = w1.shape[0] // self.epr
        h = grouped_gemm(self.x_bf16, w1, plan["row_off"], d_ff, gelu=True)
        grouped_gemm(h, w2, plan["row_off"], self.H, out=self.y)

    def combine(self, ids: torch.Tensor, probs: torch.Tensor, plan: Dict[str, torch.Tensor], out: Optional[torch.Tensor] = None,
                grouped: bool = False) -> torch.Tensor:
        """``out[t] = sum_k probs[t, k] * (expert output of assignment (t, k))``, the rows pulled over NVLink.

        ``grouped`` (after a dispatch with ``gate=probs``): every rank first adds up, locally, the weighted outputs of
        the assignments that one token has on it, and the token then pulls one row per rank instead of one per expert."""
        if out is None:
            out = torch.empty((self.T, self.H), dtype=torch.bfloat16, device="cuda")
        if grouped:
            C.moe_reduce_groups(self.y.data_ptr(), self.z.data_ptr(), self.alias.data_ptr(), self.groups.data_ptr(),
                                plan["n_rows"].data_ptr(), self.cap, self.H, torch.cuda.current_stream().cuda_stream)
            count_launch()
        self._exchange("combine", None, ids, plan["rows"], probs, out, dedupe=grouped)
        return out

    def forward(self, x: torch.Tensor, gate_logits: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
        ids, probs, plan = self.route_and_plan(gate_logits)
        self.dispatch(x, ids, plan, gate=probs)
        self.experts(w1, w2, plan)
        return self.combine(ids, probs, plan, grouped=True)
