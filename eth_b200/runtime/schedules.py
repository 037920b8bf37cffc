"""Pipeline schedules over explicit forward / backward steps.

`forward_backward_no_pipelining` and the non-interleaved 1F1B schedule
(reference: eth/runtime/megatron/schedules.py:236-281 and :595-713). A stage runs
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


def forward_only(engine, num_microbatches: int) -> None:
    """Evaluation pass: forwards only, activations dropped at once (reference: schedules.py
    `forward_only=True` branches of the same schedules)."""
    ps, comm = engine.pstate, engine.comm
    for i in range(num_microbatches):
        inputs = comm.recv_forward() if ps.num_stages > 1 else None
        out = engine.forward_step(i, inputs)
        engine.stage.drop_context(i)
        if ps.num_stages > 1:
            comm.send_forward(out)
