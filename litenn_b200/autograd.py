"""Reverse pass over the dynamic tape (the contract of litenn/core/backward.py:8-158).

Tensors are processed in descending creation order; each grad function adds into the
lazily created zero gradient of its input; branches that cannot reach a trainable tensor
are pruned unless grad_for_non_trainables; gradients of non-trainable intermediates are
released as soon as they have been consumed.
"""
import heapq

from . import ops
from .tensor import Tensor_from_value


def backward(loss, stop_grad=None, grad_for_non_trainables=False, keep_gradient_for_non_trainables=False):
    loss_gradients = {}
    if isinstance(loss, dict):
        loss_gradients = loss
        loss = list(loss.keys())
    elif not isinstance(loss, (tuple, list)):
        loss = [loss]
    if stop_grad is None:
        stop_grad = []
    elif not isinstance(stop_grad, (tuple, list)):
        stop_grad = [stop_grad]
    user_stop = set(t._get_seq_id() for t in stop_grad)

    # ---- which tensors lead to a trainable leaf? ----------------------------------------
    # `blocked` holds sequence ids through which no gradient has to flow.
    blocked = set()
    if not grad_for_non_trainables:
        reaches = {}            # seq id -> True if a trainable tensor is reachable

        def visit(t):
            t = t._get_top_reference_source() if t._is_reference() else t
            sid = t._get_seq_id()
            if sid in reaches:
                return reaches[sid]
            reaches[sid] = False          # cycle guard; the tape is a DAG
            r = t._is_trainable()
            if not r:
                for inp in t._tape_inputs():
                    if visit(inp):
                        r = True
            reaches[sid] = r
            return r

        # iterative-friendly depth: tapes here are shallow (tens of ops)
        import sys
        old = sys.getrecursionlimit()
        sys.setrecursionlimit(max(old, 100000))
        try:
            for t in loss:
                visit(t)
        finally:
            sys.setrecursionlimit(old)
        blocked = set(sid for sid, r in reaches.items() if not r)
    blocked |= user_stop

    loss_list = [t for t in loss if t._get_seq_id() not in blocked]

    # ---- seed -------------------------------------------------------------------------
    for t in loss_list:
        g = t.get_grad()
        if t in loss_gradients:
            ops.add_op(g, Tensor_from_value(loss_gradients[t]), output_t=g)
        else:
            ops.add_const_op(g, 1.0, output_t=g)

    # ---- walk: max-heap on sequence id ---------------------------------------------------
    heap, queued = [], set()

    def push(t):
        t = t._get_top_reference_source() if t._is_reference() else t
        sid = t._get_seq_id()
        if sid not in queued:
            queued.add(sid)
            heapq.heappush(heap, (-sid, id(t), t))

    for t in loss_list:
        push(t)

    while heap:
        _, _, t = heapq.heappop(heap)
        fns = t._get_gradfns()
        if fns is not None:
            for input_t, funcs in fns.items():
                if t._is_freezed() and input_t._is_trainable():
                    continue
                if input_t._get_seq_id() in blocked:
                    continue
                for func in funcs:
                    func(t, t.get_grad())
                push(input_t)
        if not grad_for_non_trainables and not t._is_trainable() and not keep_gradient_for_non_trainables:
            t.free_grad()
