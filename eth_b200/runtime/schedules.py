"""Pipeline schedules over explicit forward / backward steps.

`forward_backward_no_pipelining`, the non-interleaved 1F1B schedule and the interleaved 1F1B
schedule (reference: eth/runtime/megatron/schedules.py:236-281, :595-713 and :284-584). A stage runs
`min(stages_behind, num_microbatches)` warm-up forwards, then alternates one forward with one
backward, then drains the remaining backwards. Sends and receives that can proceed together are
issued as one batched isend/irecv, and nothing here synchronizes the host.
"""
from __future__ import annotations


def forward_backward_no_pipelining(engine, num_microbatches: int) -> None:
    for i in range(num_microbatches):
        engine.forward_step(i, None)
        engine.backward_step(i, None)


def forward_backward_1f1b(engine, num_microbatches: int) -> None:
    ps, comm = engine.pstate, engine.comm
    warmup = min(ps.num_stages - ps.stage_id - 1, num_microbatches)
    steady = num_microbatches - warmup
    t = engine.timers
    for i in range(warmup):
        inputs = comm.recv_forward()
        out = engine.forward_step(i, inputs)
        comm.send_forward(out)
    inputs = comm.recv_forward() if steady > 0 else None
    for i in range(steady):
        out = engine.forward_step(warmup + i, inputs)
        grads = comm.send_forward_recv_backward(out)
        gin = engine.backward_step(i, grads)
        if i == steady - 1:
            comm.send_backward(gin)
        else:
            inputs = comm.send_backward_recv_forward(gin)
    for i in range(warmup):
        grads = comm.recv_backward()
        gin = engine.backward_step(steady + i, grads)
        comm.send_backward(gin)
    del t


def interleaved_order(num_microbatches: int, stages: int, chunks: int):
    """The order in which a rank visits (model chunk, micro-batch) pairs, forward and backward.
    Micro-batches are taken in groups of `stages`; within a group every chunk is run for the whole
    group before the next chunk starts. Forward walks the chunks upward, backward downward."""
    if num_microbatches % stages:
        raise ValueError("interleaved pipelining needs a number of micro-batches divisible by the number of stages")
    fwd, bwd = [], []
    for group in range(num_microbatches // stages):
        for c in range(chunks):
            for j in range(stages):
                fwd.append((c, group * stages + j))
                bwd.append((chunks - 1 - c, group * stages + j))
    return fwd, bwd


def forward_backward_interleaved(engine, num_microbatches: int) -> None:
    """Interleaved 1F1B: every rank holds `chunks` model chunks, virtual stage c * S + s being chunk
    c of stage s, which shortens the pipeline bubble by the factor `chunks` at the price of `chunks`
    times as many (smaller) transfers. A rank runs (S - s - 1) * 2 + (chunks - 1) * S warm-up
    forwards, then alternates one forward with one backward, then drains. Every step posts its
    sends and the receives the *next* step needs in one batched call (`p2p.exchange`), in the same
    order on all ranks."""
    from ..parallel.p2p import exchange
    ps, comms = engine.pstate, engine.chunk_comms
    S, V, s = ps.num_stages, ps.interleave, ps.stage_id
    fwd_order, bwd_order = interleaved_order(num_microbatches, S, V)
    total = len(fwd_order)
    warmup = total if num_microbatches == S else min(total, (S - s - 1) * 2 + (V - 1) * S)
    steady = total - warmup
    inputs = [[] for _ in range(V)]       # received activations per chunk, in arrival order
    out_grads = [[] for _ in range(V)]    # received output gradients per chunk

    def run_forward(k):
        c, mb = fwd_order[k]
        feed = None if ps.is_first_virtual(c) else inputs[c].pop(0)
        return c, engine.forward_step(mb, feed, chunk=c)

    def run_backward(k):
        c, mb = bwd_order[k]
        grads = None if ps.is_last_virtual(c) else out_grads[c].pop(0)
        return c, engine.backward_step(mb, grads, chunk=c)

    def next_forward_chunk(k):
        """Chunk whose input arrives with step k's exchange (None: nothing to receive)."""
        if k + 1 >= total:
            return None
        c = fwd_order[k + 1][0]
        return None if ps.is_first_virtual(c) else c

    def next_backward_chunk(k):
        if k + 1 >= total:
            return None
        c = bwd_order[k + 1][0]
        return None if ps.is_last_virtual(c) else c

    # the input of the very first forward
    c0 = fwd_order[0][0]
    if not ps.is_first_virtual(c0):
        got, _ = exchange(recv_prev=comms[c0])
        inputs[c0].append(got)
    for k in range(warmup):
        c, out = run_forward(k)
        send = None if ps.is_last_virtual(c) else (comms[c], out)
        nf = next_forward_chunk(k)
        recv_grad = None
        if k == warmup - 1 and steady > 0:
            # the first backward of the steady phase needs its output gradient
            cb = bwd_order[0][0]
            recv_grad = None if ps.is_last_virtual(cb) else cb
        got_f, got_b = exchange(send_next=send, recv_prev=comms[nf] if nf is not None else None,
                                recv_next=comms[recv_grad] if recv_grad is not None else None)
        if nf is not None:
            inputs[nf].append(got_f)
        if recv_grad is not None:
            out_grads[recv_grad].append(got_b)
    for k in range(steady):
        fk, bk = warmup + k, k
        c, out = run_forward(fk)
        cb, gin = run_backward(bk)
        send_f = None if ps.is_last_virtual(c) else (comms[c], out)
        send_b = None if ps.is_first_virtual(cb) else (comms[cb], gin)
        nf, nb = next_forward_chunk(fk), next_backward_chunk(bk)
        got_f, got_b = exchange(send_next=send_f, send_prev=send_b, recv_prev=comms[nf] if nf is not None else None,
                                recv_next=comms[nb] if nb is not None else None)
        if nf is not None:
            inputs[nf].append(got_f)
        if nb is not None:
            out_grads[nb].append(got_b)
    if steady == 0:
        cb = bwd_order[0][0]
        if not ps.is_last_virtual(cb):
            _, got_b = exchange(recv_next=comms[cb])
            out_grads[cb].append(got_b)
    for k in range(steady, total):
        cb, gin = run_backward(k)
        send_b = None if ps.is_first_virtual(cb) else (comms[cb], gin)
        nb = next_backward_chunk(k)
        _, got_b = exchange(send_prev=send_b, recv_next=comms[nb] if nb is not None else None)
        if nb is not None:
            out_grads[nb].append(got_b)


def forward_only(engine, num_microbatches: int) -> None:
    """Evaluation pass: forwards only, activations dropped at once (reference: schedules.py
    `forward_only=True` branches of the same schedules)."""
    ps, comm = engine.pstate, getattr(engine, "eval_comm", None) or engine.comm
    for i in range(num_microbatches):
        inputs = comm.recv_forward() if ps.num_stages > 1 else None
        out = engine.forward_step(i, inputs)
        engine.stage.drop_context(i)
        if ps.num_stages > 1:
            comm.send_forward(out)
