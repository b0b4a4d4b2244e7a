"""Host-side checks of a rank's step program: the orderings that the runtime's buffers rely on.

The runtime reuses memory on purpose: CUDA-graph static buffers are shared by the micro-batches
of a (stage, slot), receive buffers are persistent per (edge, micro-batch), gradients are read
where the backward left them.  Each reuse is safe because of an ordering inside the step
program; ``program_hazards`` replays a program (no device involved) and reports every place
where such an ordering does not hold, and ``replay_job`` replays all ranks together under the
transports' semantics (sends never block, a receive waits for its send, channels are FIFO) to
show that the job terminates.  The reference has no such check (its buffers are guarded only
by waiting for outstanding sends at the end of a step, pfeife/mp/worker.py:569-574).
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

from ..parallel.schedule import Step, StepWork


def program_hazards(steps: Sequence[Step], slot_of: Dict[Tuple[int, int], int] = None
                    ) -> List[str]:
    """Problems of ONE rank's program (empty list = none):

    * a forward / backward that runs before the receive its program lists for it, or a send
      before the work that produces what it sends;
    * a backward without its forward, or anything after the optimizer step;
    * two micro-batches of a stage sharing a graph slot while both are in flight (the second
      forward would overwrite the activations the first backward still needs)."""
    out: List[str] = []
    pos: Dict[Tuple[int, int, int], int] = {}
    for i, st in enumerate(steps):
        key = (int(st.work), st.node_id, st.batch_id)
        if key in pos and st.work != StepWork.OPTIMIZER_STEP:
            out.append(f"step {i}: {st} appears twice")
        pos[key] = i
    opt = [i for i, st in enumerate(steps) if st.work == StepWork.OPTIMIZER_STEP]
    if opt and opt[0] != len(steps) - 1:
        out.append(f"step {opt[0]}: work is scheduled after the optimizer step")

    def before(a: Tuple[int, int, int], b: Tuple[int, int, int], what: str) -> None:
        if a in pos and b in pos and pos[a] > pos[b]:
            out.append(f"step {pos[b]}: {steps[pos[b]]} runs before {steps[pos[a]]} ({what})")

    for (w, s, b), i in pos.items():
        if w == StepWork.FORWARD:
            before((int(StepWork.RECV_ACT), s, b), (w, s, b), "its inputs are not there yet")
            before((w, s, b), (int(StepWork.SEND_ACT), s, b), "nothing to send yet")
        elif w == StepWork.BACKWARD:
            if (int(StepWork.FORWARD), s, b) not in pos:
                out.append(f"step {i}: {steps[i]} has no forward")
            before((int(StepWork.FORWARD), s, b), (w, s, b), "backward before forward")
            before((int(StepWork.RECV_GRAD), s, b), (w, s, b), "its gradients are not there yet")
            before((w, s, b), (int(StepWork.SEND_GRAD), s, b), "nothing to send yet")
    if slot_of:
        holder: Dict[Tuple[int, int], int] = {}      # (stage, slot) -> micro-batch in flight
        for i, st in enumerate(steps):
            if st.work == StepWork.FORWARD:
                k = (st.node_id, slot_of.get((st.node_id, st.batch_id), 0))
                if k in holder:
                    out.append(f"step {i}: {st} takes slot {k[1]} of stage {k[0]} while "
                               f"micro-batch {holder[k]} still holds it")
                holder[k] = st.batch_id
            elif st.work == StepWork.BACKWARD:
                k = (st.node_id, slot_of.get((st.node_id, st.batch_id), 0))
                if holder.get(k) == st.batch_id:
                    del holder[k]
    return out


def replay_job(programs: Sequence[Sequence[Step]], stage_rank: Dict[int, int],
               edges: Sequence[Tuple[int, int]]) -> List[str]:
    """Replays every rank's program together.  ``stage_rank[s]`` is the rank of stage s and
    ``edges`` the (producer stage, consumer stage) pairs whose values cross ranks.  A SEND step
    posts one message per consumer (activations) or producer (gradients) on the directed
    channel to that rank; a RECV step takes, in FIFO order, the messages of that (stage,
    micro-batch) and waits until they were posted.  Returns the problems found: a message
    received out of channel order, or ranks that wait for ever."""
    out: List[str] = []
    n = len(programs)
    chan: Dict[Tuple[int, int], List[Tuple[int, int, int, int]]] = {}   # (src, dst) -> queue
    cons: Dict[int, List[int]] = {}
    prod: Dict[int, List[int]] = {}
    for a, b in edges:
        if stage_rank[a] != stage_rank[b]:
            cons.setdefault(a, []).append(b)
            prod.setdefault(b, []).append(a)
    pc = [0] * n
    progressed = True
    while progressed:
        progressed = False
        for r in range(n):
            while pc[r] < len(programs[r]):
                st = programs[r][pc[r]]
                s, b = st.node_id, st.batch_id
                if st.work == StepWork.SEND_ACT:
                    for c in cons.get(s, []):
                        chan.setdefault((r, stage_rank[c]), []).append((0, s, c, b))
                elif st.work == StepWork.SEND_GRAD:
                    for p in prod.get(s, []):
                        chan.setdefault((r, stage_rank[p]), []).append((1, s, p, b))
                elif st.work in (StepWork.RECV_ACT, StepWork.RECV_GRAD):
                    grad = int(st.work == StepWork.RECV_GRAD)
                    srcs = (cons if grad else prod).get(s, [])
                    need = [(grad, q, s, b) for q in srcs]
                    ready = all(any(m == msg for m in chan.get((stage_rank[msg[1]], r), []))
                                for msg in need)
                    if not ready:
                        break
                    for msg in need:
                        q = chan[(stage_rank[msg[1]], r)]
                        # everything ahead of it on the channel must belong to a receive this
                        # rank has already posted or will post first: with per-message buffers
                        # only the ORDER of consumption per channel has to match
                        q.remove(msg)
                pc[r] += 1
                progressed = True
    for r in range(n):
        if pc[r] < len(programs[r]):
            out.append(f"rank {r} waits for ever at step {pc[r]}: {programs[r][pc[r]]}")
    for k, q in chan.items():
        if q:
            out.append(f"channel {k[0]}->{k[1]}: {len(q)} message(s) never received")
    return out
