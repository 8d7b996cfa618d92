"""Feed-forward parts: the dense SwiGLU MLP and the sparse mixture of SwiGLU experts with a
softmax router, top-k routing and an optional sigmoid-gated shared expert."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, RowMix, TensorSpec
from .linear import linear, grouped_linear, small_linear
from .registry import register_part

# Batches of up to this many rows run the shared expert's chunks on a second stream beside the routing.
SIDE_MAX_ROWS = 64
# Prompts: the shared expert's two products run beside the routing chain (router product, top-k, permutation, row
# copy) on a second stream with their grid capped to this share of the multiprocessors, which leaves the chain's
# kernels room; the routed experts' products follow on the first stream.
SIDE_GRID_SHARE = 0.88
# Permutation buffers are kept per batch size; beyond this many sizes the oldest set is dropped.
MAX_ALIGNMENTS = 16


class DenseSwiGLU(FeedForward):
    """``down(silu(gate(h)) * up(h))`` (src/model.cpp:828-832; src/hip_ops.hip:419-429)."""

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden, self.inter = hidden_size, intermediate_size

    def tensor_specs(self, available=None):
        H, I = self.hidden, self.inter
        return {"gate_proj.weight": TensorSpec((I, H)), "up_proj.weight": TensorSpec((I, H)),
                "down_proj.weight": TensorSpec((H, I))}

    def load(self, fetch, ctx):
        self.ctx = ctx
        # gate rows then up rows in one matrix (src/model.cpp:589-596)
        self.gate_up = _cat([fetch("gate_proj.weight"), fetch("up_proj.weight")])
        self.down = fetch("down_proj.weight")

    def forward(self, h, h32, batch):
        act = linear(self.ctx, h, self.gate_up, self.ctx.act_dtype, swiglu=True)
        return linear(self.ctx, act, self.down, torch.float32)


class SparseMoeSwiGLU(FeedForward):
    """Per row (src/model.cpp:789-827; src/hip_ops.hip:813-893, 926-934):

    router logits ``r = h Wg^T`` in float32; ``p = softmax(r)`` over all experts; the ``top_k``
    largest (ties to the lower index) with weights ``p`` or ``p / sum`` (``renormalize``);
    ``routed = sum_k w_k * down_e(silu(gate_e(h)) * up_e(h))`` for k in rank order;
    ``shared = sigmoid(h . w_gate) * down_s(silu(gate_s(h)) * up_s(h))`` if there is a shared
    expert; the result is ``shared + routed``.
    """
    wants_f32_input = True

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, intermediate_size: int,
                 shared_intermediate_size: int = 0, renormalize: bool = False):
        if not (1 <= top_k <= num_experts):
            raise ValueError("top_k must lie in 1..num_experts")
        if top_k > 32 or num_experts > 1536:
            raise ValueError("the router kernel takes up to 32 experts per row out of up to 1536")
        self.hidden, self.E, self.K = hidden_size, num_experts, top_k
        self.inter, self.shared_inter, self.renorm = intermediate_size, shared_intermediate_size, renormalize
        self._align = {}
        self._counters = None
        self._captured = {}
        self._static = {}
        self._static_kept = set()
        self.router_and_gate = None
        self.last_alignment = None      # the permutation buffers of the latest forward (for statistics)

    def tensor_specs(self, available=None):
        H, I, E, SI = self.hidden, self.inter, self.E, self.shared_inter
        s = {"gate.weight": TensorSpec((E, H))}
        if available is not None and available("experts.gate_up_proj"):  # stacked form, src/model.cpp:274-281
            s["experts.gate_up_proj"] = TensorSpec((E, 2 * I, H))
            s["experts.down_proj"] = TensorSpec((E, H, I))
        else:
            for e in range(E):
                s[f"experts.{e}.gate_proj.weight"] = TensorSpec((I, H))
                s[f"experts.{e}.up_proj.weight"] = TensorSpec((I, H))
                s[f"experts.{e}.down_proj.weight"] = TensorSpec((H, I))
        if SI > 0:
            s["shared_expert.gate_proj.weight"] = TensorSpec((SI, H))
            s["shared_expert.up_proj.weight"] = TensorSpec((SI, H))
            s["shared_expert.down_proj.weight"] = TensorSpec((H, SI))
            s["shared_expert_gate.weight"] = TensorSpec((1, H))
        return s

    def load(self, fetch, ctx):
        self.ctx = ctx
        H, I, E, SI = self.hidden, self.inter, self.E, self.shared_inter
        self.router = fetch("gate.weight")
        stacked = fetch.has("experts.gate_up_proj")
        first = fetch("experts.gate_up_proj") if stacked else fetch("experts.0.gate_proj.weight")
        # The shared expert as C more experts that every row visits: possible when its width is a whole
        # number of expert widths.  Its chunks then ride in the grouped products and need no launches of
        # their own.  Only the tensor-core path does this; the plain path keeps the shared expert apart.
        C = SI // I if (SI > 0 and SI % I == 0 and SI // I <= 32) else 0
        self.virtual = C if (ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and first.dtype == torch.bfloat16
                             and H % 8 == 0 and I % 8 == 0) else 0
        EC = E + self.virtual
        # every expert's [gate; up] rows and down matrix in one block each, indexed by expert
        self.w_gate_up = torch.empty((EC, 2 * I, H), dtype=first.dtype, device=first.device)
        self.w_down = torch.empty((EC, H, I), dtype=first.dtype, device=first.device)
        if stacked:
            self.w_gate_up[:E].copy_(first)
            self.w_down[:E].copy_(fetch("experts.down_proj"))
        else:
            for e in range(E):
                self.w_gate_up[e, :I].copy_(first if e == 0 else fetch(f"experts.{e}.gate_proj.weight"))
                self.w_gate_up[e, I:].copy_(fetch(f"experts.{e}.up_proj.weight"))
                self.w_down[e].copy_(fetch(f"experts.{e}.down_proj.weight"))
        del first
        if SI > 0:
            sg, su = fetch("shared_expert.gate_proj.weight"), fetch("shared_expert.up_proj.weight")
            sd = fetch("shared_expert.down_proj.weight")
            self.sh_gate = fetch("shared_expert_gate.weight")
            # the gate's single row rides along with the router's rows: one product gives both logits
            if self.sh_gate.dtype == self.router.dtype:
                self.router_and_gate = torch.cat([self.router, self.sh_gate.reshape(1, -1)], dim=0).contiguous()
            if self.virtual and sg.dtype == su.dtype == sd.dtype == self.w_gate_up.dtype and self.router_and_gate is not None:
                for c in range(self.virtual):
                    self.w_gate_up[E + c, :I].copy_(sg[c * I:(c + 1) * I])
                    self.w_gate_up[E + c, I:].copy_(su[c * I:(c + 1) * I])
                    self.w_down[E + c].copy_(sd[:, c * I:(c + 1) * I])
            else:
                if self.virtual:                       # mixed storage types: keep the shared expert apart
                    self.w_gate_up, self.w_down = self.w_gate_up[:E].clone(), self.w_down[:E].clone()
                    self.virtual = 0
                self.sh_gate_up = _cat([sg, su])
                self.sh_down = sd
        else:
            self.virtual = 0

    def _alignment(self, TK, n_experts, device, fast):
        if fast:    # the down product's tile is the primary list, the SwiGLU product may want a wider one
            tile_m, tile_m2 = ops.grouped_token_tile(TK, n_experts), ops.grouped_token_tile(TK, n_experts, swiglu=True)
        else:
            tile_m, tile_m2 = ops.gemm_plain_tile_m(), 0
        key = (TK, n_experts, tile_m, tile_m2)
        if key in self._captured:
            return self._captured[key]
        al = self._align.pop(key, None)
        if al is None:
            if len(self._align) >= MAX_ALIGNMENTS:
                self._align.pop(next(iter(self._align)))
            al = ops.MoeAlignment(TK, n_experts, tile_m, device, tile_m2)
        if torch.cuda.is_current_stream_capturing():     # a captured step names these buffers by address: kept for good
            self._captured[key] = al
        else:
            self._align[key] = al                        # most recently used last
        return al

    def forward(self, h, h32, batch):
        ctx = self.ctx
        T = h.shape[0]
        dev = h.device
        C = self.virtual
        KT = self.K + C
        gate_logit = None
        if self.router_and_gate is not None:
            both = small_linear(ctx, h32, self.router_and_gate)
            logits, gate_logit = both[:, :self.E], both[:, self.E:]
        else:
            logits = small_linear(ctx, h32, self.router)
        idx = torch.empty((T, KT), dtype=torch.int32, device=dev)
        score = torch.empty((T, KT), dtype=torch.float32, device=dev)
        fast = (ctx.fast_kernels and h.dtype == torch.bfloat16 and self.w_gate_up.dtype == torch.bfloat16
                and self.w_down.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inter % 8 == 0)
        al = self._alignment(T * KT, self.E + C, dev, fast)
        x_sorted = None
        if (fast and C and T <= SIDE_MAX_ROWS and al.secondary is None
                and ops.moe_route_small_usable(T, self.E, self.K, C, self.hidden)):
            return self._forward_beside(h, logits, gate_logit, idx, score, al)
        if fast and C and T >= 256 and al.secondary is None:
            return self._forward_beside(h, logits, gate_logit, idx, score, al, many=True)
        # (the products' CTAs take their tiles from a counter, as in _forward_beside, unless a handful of pairs split K)
        c0 = c1 = zero = None
        if fast and al.TK > ops.GROUPED_SPLIT_MAX_PAIRS:
            if self._counters is None:
                self._counters = torch.zeros(2, dtype=torch.int32, device=dev)
            zero, c0, c1 = self._counters, self._counters[0:1], self._counters[1:2]
        if fast and al.secondary is None and ops.moe_route_small_usable(T, self.E, self.K, C, self.hidden):
            x_sorted = ops.moe_route_small(logits, self.K, self.renorm, C, gate_logit, idx, score, al, ctx.err,
                                           x=None, zero=zero)   # one block copies rows slower than the copy kernel does
        else:
            ops.router_topk(logits, self.K, self.renorm, idx, score, C, gate_logit)
            ops.moe_align(idx, KT, al, ctx.err, spread_last=C if fast else 0, zero=zero)
        self.last_alignment = al
        wide = al.secondary                      # the tile list of the SwiGLU product, if it has one of its own
        if x_sorted is not None:
            act = grouped_linear(ctx, x_sorted, self.w_gate_up, ctx.act_dtype, al, swiglu=True, tiles=wide, counter=c0)
        else:
            act = grouped_linear(ctx, h, self.w_gate_up, ctx.act_dtype, al, a_rows=al.sorted_token, swiglu=True,
                                 tiles=wide, counter=c0)
        # the tile lists were final before the first product started: the second may start beside it
        y = grouped_linear(ctx, act, self.w_down, torch.float32, al, tiles_ready=True, counter=c1)
        shared = None
        if self.shared_inter > 0 and not C:
            sact = linear(ctx, h, self.sh_gate_up, ctx.act_dtype, swiglu=True)
            shared = linear(ctx, sact, self.sh_down, torch.float32)
            if gate_logit is None:
                gate_logit = small_linear(ctx, h32, self.sh_gate)
        # the combination (src/hip_ops.hip:873-892) is left to whoever takes the branch: the next norm sums it
        return RowMix(y, al.pair_pos[:T * KT].view(T, KT), score, shared, gate_logit if shared is not None else None)


    def _forward_beside(self, h, logits, gate_logit, idx, score, al, many=False):
        """The shared expert's chunks need no routing, so their two products run on a second stream beside the
        routing and the row copy, which keep few multiprocessors busy; the routed experts' products follow on the
        first stream and write the other rows of the same two buffers.  Few rows (decoding): one launch routes.
        ``many`` rows (a prompt): the routing is three kernels that take a tenth of the layer's time, and the side
        products leave them some multiprocessors."""
        ctx, T, K, C, dev = self.ctx, h.shape[0], self.K, self.virtual, h.device
        KT = K + C
        key = (T, dev)
        st = self._static.get(key)
        if st is None:
            loose = [k for k in self._static if k not in self._static_kept]
            if len(loose) >= MAX_ALIGNMENTS:
                self._static.pop(loose[0])
            st = self._static[key] = ops.StaticTiles(T, K, self.E, C, dev)
        if torch.cuda.is_current_stream_capturing():       # a captured step names these buffers by address
            self._static_kept.add(key)
        act = torch.empty((T * KT, self.inter), dtype=ctx.act_dtype, device=dev)
        y = torch.empty((T * KT, self.hidden), dtype=torch.float32, device=dev)
        main, side = torch.cuda.current_stream(dev), _side_stream(dev)
        fork, join = torch.cuda.Event(), torch.cuda.Event()
        fork.record(main)
        side.wait_event(fork)
        cap = int(ops.num_sms() * SIDE_GRID_SHARE) if many else 0
        with torch.cuda.stream(side):
            ops.gemm_fast_grouped(h, self.w_gate_up, act, al, swiglu=True, err=ctx.err, tiles=st, tiles_ready=True,
                                  x_rows=st.x_rows, max_ctas=cap)
            ops.gemm_fast_grouped(act, self.w_down, y, al, err=ctx.err, tiles=st, tiles_ready=True, max_ctas=cap)
            join.record(side)
        # The routed products' CTAs take their tiles from a counter: a prompt's start while the side products still hold
        # most multiprocessors, so the ones that start early do more of the work; a decode step's tiles are one to
        # three per CTA, and CTAs that are through with theirs take what is left (measured per decode step: batch 8
        # 3.70 -> 3.63 ms, batch 16 5.42 -> 5.23, batch 32 7.77 -> 7.52, batch 64 10.24 -> 10.18).  A handful of pairs
        # go without: their products split K instead.  A product sets its counter back itself; one that gave up on a
        # wait may not have, so the routing kernel zeroes both.
        c0 = c1 = None
        if many or al.TK > ops.GROUPED_SPLIT_MAX_PAIRS:
            if self._counters is None:
                self._counters = torch.zeros(2, dtype=torch.int32, device=dev)
            c0, c1 = self._counters[0:1], self._counters[1:2]
        if many:
            ops.router_topk(logits, K, self.renorm, idx, score, C, gate_logit)
            ops.moe_align(idx, KT, al, ctx.err, static_last=C, zero=self._counters)
        else:
            ops.moe_route_small(logits, K, self.renorm, C, gate_logit, idx, score, al, ctx.err, x=None, static=True,
                                zero=self._counters if c0 is not None else None)
        self.last_alignment = al
        x_sorted = ops.permute_rows(h, al.sorted_token, T * K)
        ops.gemm_fast_grouped(x_sorted, self.w_gate_up, act, al, swiglu=True, err=ctx.err, tiles_ready=True, counter=c0)
        ops.gemm_fast_grouped(act, self.w_down, y, al, err=ctx.err, tiles_ready=True, counter=c1)
        main.wait_event(join)
        return RowMix(y, al.pair_pos[:T * KT].view(T, KT), score, None, None)


_side = {}


def _side_stream(dev):
    """One second stream per device for work that runs beside a step's main stream."""
    if ops.timing():                 # per-kernel timers are running: one stream, one kernel after the other
        return torch.cuda.current_stream(dev)
    key = torch.device(dev)
    if key not in _side:
        _side[key] = torch.cuda.Stream(device=key)
    return _side[key]


def _cat(ts):
    if len({t.dtype for t in ts}) > 1:
        ts = [t.float() for t in ts]
    return torch.cat(ts, dim=0).contiguous()


register_part("feed_forward", "dense_swiglu", DenseSwiGLU)
register_part("feed_forward", "sparse_moe_swiglu", SparseMoeSwiGLU)
