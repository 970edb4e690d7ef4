"""Forward/backward overlap for MoE layers: hide the dispatch / combine all-to-alls of one micro-batch under the
attention / expert compute of another.

A transformer layer with a routed MLP is cut into four stages

      attention      norm + self-attention + residual                       (compute)
      dispatch       norm + router + permute + all-to-all                   (communication)
      experts        grouped expert MLP (+ shared expert)                   (compute)
      combine        all-to-all + un-permute + residual                     (communication)

and every stage is its own autograd sub-graph: its inputs are detached leaves, its outputs are kept in a
``LayerGraph``.  Backward walks the stages in reverse, feeding each stage the gradient of its outputs and reading
the gradients of its detached inputs - so a forward stage of micro-batch i and a backward stage of micro-batch j
are independent pieces of work that can be issued alternately on a compute stream and a communication stream:

      compute stream :  F.attention(i)      B.experts(j)        F.experts(i)        B.attention(j)
      comm stream    :  B.combine(j)        F.dispatch(i)       B.dispatch(j)       F.combine(i)

(the four forward x backward pairings of the reference collapse into this one table; a dense layer simply has empty
communication stages).  Weight gradients of the compute stages can be deferred through ``WeightGradStore`` by the
caller so that pipeline sends hide under them.
reference: mindspeed/core/transformer/moe/moe_feature/fb_overlap/modules/utils.py:80-130 (LayerGraph),
overlap_funcs/fwdbwd.py:37,381,684,845 (stage interleavings), vpp_schedules.py:300-990 (schedule integration).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch

STAGES = ("attention", "dispatch", "experts", "combine")


def _detach_leaf(t):
    if isinstance(t, torch.Tensor) and t.is_floating_point():
        return t.detach().requires_grad_(True)
    return t


class _StageRecord:
    __slots__ = ("inputs", "outputs")

    def __init__(self, inputs, outputs):
        self.inputs, self.outputs = inputs, outputs


class LayerGraph:
    """The detached stage sub-graphs of one layer call; ``backward_stage`` consumes them in reverse order."""

    def __init__(self):
        self.records: List[_StageRecord] = []
        self.pending_grads: Optional[Tuple] = None

    def run_stage(self, fn: Callable, inputs: Sequence):
        leaves = tuple(_detach_leaf(t) for t in inputs)
        with torch.enable_grad():
            outs = fn(*leaves)
        outs = outs if isinstance(outs, tuple) else (outs,)
        self.records.append(_StageRecord(leaves, outs))
        return tuple(o.detach() if isinstance(o, torch.Tensor) else o for o in outs)

    def backward_stage(self, grads: Sequence[Optional[torch.Tensor]]) -> Tuple:
        rec = self.records.pop()
        pairs = [(o, g) for o, g in zip(rec.outputs, grads)
                 if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([p[0] for p in pairs], [p[1] for p in pairs])
        return tuple(t.grad if isinstance(t, torch.Tensor) and t.requires_grad else None for t in rec.inputs)

    @property
    def stages_left(self) -> int:
        return len(self.records)


class StagedMoELayer:
    """The four stage functions of a ``TransformerLayer`` whose ``mlp`` is a ``MoELayer`` (or a dense MLP)."""

    def __init__(self, layer):
        self.layer = layer
        self.is_moe = hasattr(layer.mlp, "token_dispatcher")
        self._ctx = {}

    # stage signatures: tensors in, tensors out (non-tensor context is kept on self._ctx per call id)
    def attention(self, hidden, **kw):
        L = self.layer
        ln = L.input_layernorm(hidden)
        out, bias = L.self_attention(ln, **kw)
        if bias is not None:
            out = out + bias
        return hidden + out

    def dispatch(self, hidden):
        L = self.layer
        ln = L.pre_mlp_layernorm(hidden)
        if not self.is_moe:
            return hidden, ln
        moe = L.mlp
        probs, routing_map = moe.router(ln)
        rows, tpe, row_probs = moe.token_dispatcher.token_permutation(ln, probs.to(ln.dtype), routing_map)
        self._ctx["tpe"] = tpe
        self._ctx["snapshot"] = _snapshot_dispatcher(moe.token_dispatcher)
        return hidden, ln, rows, row_probs

    def experts(self, hidden, ln, rows=None, row_probs=None):
        L = self.layer
        if not self.is_moe:
            out, bias = L.mlp(ln)
            return hidden, (out if bias is None else out + bias)
        moe = L.mlp
        y, _ = moe.experts(rows, self._ctx["tpe"], row_probs)
        shared = moe.shared_experts(ln) if moe.shared_experts is not None else None
        return (hidden, y, shared) if shared is not None else (hidden, y)

    def combine(self, hidden, y, shared=None):
        if not self.is_moe:
            return hidden + y
        moe = self.layer.mlp
        _restore_dispatcher(moe.token_dispatcher, self._ctx["snapshot"])
        out, _ = moe.token_dispatcher.token_unpermutation(y)
        if shared is not None:
            out = out + shared
        return hidden + out

    def functions(self, **attn_kw):
        return [lambda h: self.attention(h, **attn_kw), self.dispatch, self.experts, self.combine]


_DISPATCHER_STATE = ("hidden_shape", "restore_shape", "sorted_indices", "input_splits", "output_splits", "chunk_sizes",
                     "routing_map", "probs", "local_map", "local_probs", "_plan", "_cap_rows", "_fused_now")


def _snapshot_dispatcher(d):
    """A dispatcher keeps per-call state on itself; interleaving two micro-batches needs it saved and restored."""
    return {k: getattr(d, k) for k in _DISPATCHER_STATE if hasattr(d, k)}


def _restore_dispatcher(d, snap):
    for k, v in snap.items():
        setattr(d, k, v)


def _tensors(xs):
    return [t for t in xs if isinstance(t, torch.Tensor)]


class _Streams:
    """The compute stream is the caller's current stream; communication stages run on a second one.

    A tensor produced on one stream and consumed on the other is recorded on the consumer's stream, so that the caching
    allocator does not hand its memory to a later allocation on the producer's stream while the consumer still reads it.
    """

    def __init__(self, device):
        self.cuda = isinstance(device, torch.device) and device.type == "cuda"
        self.comm = torch.cuda.Stream(device=device) if self.cuda else None

    def mark(self):
        """An event on the compute stream: work queued on it afterwards does not hold back ``on_comm(..., after=event)``."""
        return torch.cuda.current_stream().record_event() if self.cuda else None

    def on_comm(self, fn, inputs=(), after=None):
        """Run ``fn`` on the communication stream, ordered after ``after`` (an event from ``mark``) or, without one,
        after everything the compute stream has queued so far."""
        if not self.cuda:
            return fn()
        main = torch.cuda.current_stream()
        if after is not None:
            self.comm.wait_event(after)
        else:
            self.comm.wait_stream(main)
        for t in _tensors(inputs):
            t.record_stream(self.comm)
        with torch.cuda.stream(self.comm):
            out = fn()
        for t in _tensors(out if isinstance(out, (tuple, list)) else (out,)):
            t.record_stream(main)
        return out

    def join(self):
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm)


COMM_STAGES = (1, 3)        # dispatch and combine


def forward_layer_staged(staged: StagedMoELayer, hidden: torch.Tensor, streams: Optional[_Streams] = None,
                         **attn_kw) -> Tuple[torch.Tensor, LayerGraph]:
    """Plain (non-overlapped) staged forward; returns the detached output and the graph for a later backward.

    With ``streams`` the dispatch and combine stages run on the communication stream: autograd executes a node's backward
    on the stream of its forward, so this is what later lets their backward overlap another micro-batch's compute."""
    g = LayerGraph()
    cur: Tuple = (hidden,)
    for k, fn in enumerate(staged.functions(**attn_kw)):
        if streams is not None and k in COMM_STAGES:
            cur = streams.on_comm(lambda fn=fn, cur=cur: g.run_stage(fn, cur), cur)
            streams.join()
        else:
            cur = g.run_stage(fn, cur)
    return cur[0], g


def backward_layer_staged(graph: LayerGraph, grad_out: torch.Tensor) -> torch.Tensor:
    grads: Tuple = (grad_out,)
    while graph.stages_left:
        grads = graph.backward_stage(grads)
    return grads[0]


def forward_backward_overlapped(fwd: StagedMoELayer, hidden: torch.Tensor, bwd_graph: LayerGraph, grad_out: torch.Tensor,
                                streams: Optional[_Streams] = None, **attn_kw):
    """Forward of one micro-batch through ``fwd`` interleaved with the backward of another micro-batch's
    ``bwd_graph`` (four stages each).  Returns (forward output, forward graph, input gradient of the backward)."""
    if bwd_graph.stages_left != 4:
        raise ValueError("the backward graph must hold exactly the four stages of one layer")
    st = streams or _Streams(hidden.device)
    f_attn, f_disp, f_exp, f_comb = fwd.functions(**attn_kw)
    g = LayerGraph()
    # In every slot the piece that never blocks the host is queued first.  F.dispatch reads the split sizes back to the
    # host; queued after B.experts, that wait is spent while the GPU runs B.experts.
    # slot 1: F.attention on compute | B.combine on comm
    gb = st.on_comm(lambda: bwd_graph.backward_stage((grad_out,)), (grad_out,))
    cur = g.run_stage(f_attn, (hidden,))
    st.join()
    # slot 2: B.experts on compute | F.dispatch on comm
    ev = st.mark()                       # everything both pieces need is complete here; B.experts must not delay F.dispatch
    gb_e = bwd_graph.backward_stage(gb)
    cur2 = st.on_comm(lambda: g.run_stage(f_disp, cur), cur, after=ev)
    st.join()
    # slot 3: F.experts on compute | B.dispatch on comm
    ev = st.mark()
    cur3 = g.run_stage(f_exp, cur2)
    gb2 = st.on_comm(lambda: bwd_graph.backward_stage(gb_e), gb_e, after=ev)
    st.join()
    # slot 4: B.attention on compute | F.combine on comm
    ev = st.mark()
    gin = bwd_graph.backward_stage(gb2)
    out = st.on_comm(lambda: g.run_stage(f_comb, cur3), cur3, after=ev)
    st.join()
    return out[0], g, gin[0]


def run_microbatches_overlapped(layers: Sequence, inputs: List[torch.Tensor], grad_fn: Callable[[int, torch.Tensor], torch.Tensor],
                                **attn_kw):
    """No-pipeline driver over a stack of layers: micro-batch i's forward through layer k overlaps micro-batch i-1's
    backward through the same layer (one extra warm-up forward, one cool-down backward).

    ``grad_fn(i, output)`` returns d(loss_i)/d(output).  Returns (outputs, input gradients)."""
    staged = [StagedMoELayer(l) for l in layers]
    n = len(inputs)
    outs: List[Optional[torch.Tensor]] = [None] * n
    gins: List[Optional[torch.Tensor]] = [None] * n
    graphs: List[List[LayerGraph]] = [[] for _ in range(n)]
    # warm-up: forward of micro-batch 0
    h = inputs[0]
    for s in staged:
        h, g = forward_layer_staged(s, h, **attn_kw)
        graphs[0].append(g)
    outs[0] = h
    streams = _Streams(inputs[0].device)
    for i in range(1, n):
        # forward of i goes up the stack while backward of i-1 goes down it: layer k of F pairs with layer (L-1-k) of B
        h = inputs[i]
        grad = grad_fn(i - 1, outs[i - 1])
        for k, s in enumerate(staged):
            bg = graphs[i - 1][len(staged) - 1 - k]
            h, g, grad = forward_backward_overlapped(s, h, bg, grad, streams, **attn_kw)
            graphs[i].append(g)
        outs[i], gins[i - 1] = h, grad
    grad = grad_fn(n - 1, outs[n - 1])
    for g in reversed(graphs[n - 1]):
        grad = backward_layer_staged(g, grad)
    gins[n - 1] = grad
    return outs, gins


class BlockOverlap:
    """Forward of micro-batch i through a stack of layers interleaved with the backward of micro-batch i-1, driven from
    inside ``TransformerBlock.forward`` so that the ordinary ``forward_step`` / loss function stay unchanged.

    Per micro-batch the block keeps the staged graphs of its layers, the (attached) block input and a detached leaf as
    block output.  The loss backward of the schedule stops at that leaf; its ``.grad`` is the seed of the layer backward
    that runs interleaved with the next micro-batch's forward (or alone in ``finish``).
    reference: the 1F1B-overlap entry of mindspeed/core/transformer/moe/moe_feature/fb_overlap/overlap_funcs/fwdbwd.py:37-380
    and its scheduling in vpp_schedules.py:300-990.
    """

    def __init__(self, layers: Sequence):
        self.staged = [StagedMoELayer(l) for l in layers if hasattr(l, "mlp")]     # no-op layers are identities: left out
        self.streams: Optional[_Streams] = None
        self.prev = None          # (graphs, block input, output leaf) of the micro-batch whose backward is pending

    def forward(self, hidden: torch.Tensor, **attn_kw) -> torch.Tensor:
        if self.streams is None:
            self.streams = _Streams(hidden.device)
        graphs: List[LayerGraph] = []
        h = hidden.detach()
        if self.prev is None:
            for s in self.staged:
                h, g = forward_layer_staged(s, h, self.streams, **attn_kw)
                graphs.append(g)
        else:
            p_graphs, p_in, p_leaf = self.prev
            grad = p_leaf.grad
            if grad is None:
                raise RuntimeError("forward/backward overlap: the previous micro-batch's loss backward has not run")
            n = len(self.staged)
            for k, s in enumerate(self.staged):
                h, g, grad = forward_backward_overlapped(s, h, p_graphs[n - 1 - k], grad, self.streams, **attn_kw)
                graphs.append(g)
            self._finish_input(p_in, grad)
        leaf = h.detach().requires_grad_(True)
        self.prev = (graphs, hidden, leaf)
        return leaf

    @staticmethod
    def _finish_input(block_input, grad):
        if isinstance(block_input, torch.Tensor) and block_input.requires_grad and grad is not None:
            block_input.backward(grad)

    def finish(self):
        """Backward of the last micro-batch (nothing left to overlap with)."""
        if self.prev is None:
            return
        graphs, p_in, p_leaf = self.prev
        self.prev = None
        grad = p_leaf.grad
        if grad is None:
            return
        for g in reversed(graphs):
            grad = backward_layer_staged(g, grad)
        self._finish_input(p_in, grad)


class StagedBlockState:
    """Pipeline form of the overlap: a model chunk's layer stack keeps the staged graphs of every (chunk, micro-batch) whose
    backward is still to come, and a forward can be given a PARTNER - another chunk's pending micro-batch on the same rank -
    whose layer backward is then interleaved with it stage by stage (the F || B slots of a pipeline schedule).

        forward(key, hidden, partner=None)   staged forward; with partner = (state, key) the partner's layers run backward
                                             in between (last layer of the partner against the first layer of this one)
        backward(key)                        the layer backward of ``key`` if no forward has done it, then the gradient goes
                                             into the block input (the received activation's ``.grad`` or the embedding)
    The seed of a backward is the ``.grad`` of the detached output leaf, put there by the stage's own post-processing (loss
    backward on the last stage, ``torch.autograd.backward(output, received gradient)`` elsewhere).
    reference: mindspeed/core/transformer/moe/moe_feature/fb_overlap/vpp_schedules.py:300-990 (F || B pairing in the
    interleaved schedule) and dualpipev/dualpipev_schedules.py:310-346 (overlap phase)."""

    def __init__(self, layers: Sequence):
        self.staged = [StagedMoELayer(l) for l in layers if hasattr(l, "mlp")]     # no-op layers are identities: left out
        self.streams: Optional[_Streams] = None
        self.records = {}

    def forward(self, key, hidden: torch.Tensor, partner=None, **attn_kw) -> torch.Tensor:
        if self.streams is None:
            self.streams = _Streams(hidden.device)
        graphs: List[LayerGraph] = []
        h = hidden.detach()
        if partner is None:
            for s in self.staged:
                h, g = forward_layer_staged(s, h, self.streams, **attn_kw)
                graphs.append(g)
        else:
            pstate, pkey = partner
            p_graphs, p_in, p_leaf = pstate.records[pkey]
            grad = p_leaf.grad
            if grad is None:
                raise RuntimeError("forward/backward overlap: the partner micro-batch has no output gradient yet")
            n = min(len(self.staged), len(p_graphs))
            for k in range(n):
                h, g, grad = forward_backward_overlapped(self.staged[k], h, p_graphs[len(p_graphs) - 1 - k], grad, self.streams, **attn_kw)
                graphs.append(g)
            for s in self.staged[n:]:
                h, g = forward_layer_staged(s, h, self.streams, **attn_kw)
                graphs.append(g)
            for g in reversed(p_graphs[:len(p_graphs) - n]):
                grad = backward_layer_staged(g, grad)
            pstate.records[pkey] = (None, p_in, grad)                   # layers done: only the block input is left
        leaf = h.detach().requires_grad_(True)
        self.records[key] = (graphs, hidden, leaf)
        return leaf

    def backward(self, key):
        graphs, block_input, x = self.records.pop(key)
        if graphs is None:
            grad = x
        else:
            grad = x.grad
            if grad is None:
                return
            for g in reversed(graphs):
                grad = backward_layer_staged(g, grad)
        if isinstance(block_input, torch.Tensor) and block_input.requires_grad and grad is not None:
            block_input.backward(grad)
