"""Picture of a planned schedule: one lane per pipeline rank, one box per (stage, micro-batch,
direction) placed at the start time the planner's simulation gave it.

The reference draws the same chart with matplotlib (pfeife/schedule/planner.py:583-624,
``save_graph_png``); this one writes SVG text directly, so it needs no plotting package, and
also offers the rows as plain data (``schedule_rows``) and as a text table.
"""
from __future__ import annotations

from typing import List, NamedTuple

from .pipe_graph import PipeGraph, Simulation
from .schedule import PipeSchedParams


class Box(NamedTuple):
    rank: int
    stage: int
    batch: int
    is_fwd: bool
    start: float     # ms
    dur: float       # ms


def schedule_rows(pipe_graph: PipeGraph, sched: PipeSchedParams,
                  sim: Simulation = None) -> List[Box]:
    """Every compute item of the schedule with its simulated start and its duration, ordered by
    rank and start time."""
    if sim is None or not sim.start_times:
        sim = pipe_graph.simulate(sched, record=True)
    rows = []
    for r, works in enumerate(sched.rank_works):
        for s, b, fwd in works:
            n = pipe_graph.nodes[s]
            rows.append(Box(r, s, b, bool(fwd), float(sim.start_times[(s, b, fwd)]),
                            float(n.comp_time if fwd else n.back_time)))
    rows.sort(key=lambda x: (x.rank, x.start))
    return rows


def schedule_table(pipe_graph: PipeGraph, sched: PipeSchedParams, sim: Simulation = None) -> str:
    lines = ["rank stage batch dir   start_ms     dur_ms"]
    for x in schedule_rows(pipe_graph, sched, sim):
        lines.append(f"{x.rank:4d} {x.stage:5d} {x.batch:5d} {'fwd' if x.is_fwd else 'bwd'} "
                     f"{x.start:10.3f} {x.dur:10.3f}")
    return "\n".join(lines)


_COLORS = ("#1f77b4", "#ff7f0e", "#d62728", "#2ca02c", "#9467bd", "#8c564b", "#e377c2",
           "#17becf")


def save_schedule_svg(pipe_graph: PipeGraph, sched: PipeSchedParams, path: str,
                      sim: Simulation = None, width: int = 1400, lane: int = 44) -> str:
    """Writes the chart to `path` and returns it.  Colour = micro-batch, forward boxes are
    filled, backward boxes are hatched lighter; the label is ``stage_microbatch``."""
    if sim is None or not sim.start_times:
        sim = pipe_graph.simulate(sched, record=True)
    rows = schedule_rows(pipe_graph, sched, sim)
    ranks = len(sched.rank_works)
    end = max(max((x.start + x.dur for x in rows), default=0.0), float(sim.makespan)) or 1.0
    left, top = 70, 24
    scale = (width - left - 20) / end
    height = top + ranks * lane + 40
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" '
           f'font-family="monospace" font-size="10">',
           f'<rect width="{width}" height="{height}" fill="white"/>']
    for r in range(ranks):
        y = top + r * lane
        out.append(f'<text x="6" y="{y + lane / 2 + 3:.1f}">rank {r}</text>')
        out.append(f'<line x1="{left}" y1="{y + lane - 4}" x2="{width - 20}" y2="{y + lane - 4}" '
                   f'stroke="#cccccc"/>')
    for x in rows:
        y = top + x.rank * lane + 4
        w = max(x.dur * scale, 0.5)
        x0 = left + x.start * scale
        color = _COLORS[x.batch % len(_COLORS)]
        opacity = "1.0" if x.is_fwd else "0.55"
        out.append(f'<rect x="{x0:.2f}" y="{y}" width="{w:.2f}" height="{lane - 12}" '
                   f'fill="{color}" fill-opacity="{opacity}" stroke="black" stroke-width="0.6">'
                   f'<title>stage {x.stage} micro-batch {x.batch} '
                   f'{"forward" if x.is_fwd else "backward"}: {x.start:.3f} ms + {x.dur:.3f} ms'
                   f'</title></rect>')
        if w >= 22:
            out.append(f'<text x="{x0 + w / 2:.2f}" y="{y + (lane - 12) / 2 + 3:.1f}" '
                       f'text-anchor="middle" fill="white">{x.stage}_{x.batch}</text>')
    ticks = 10
    for i in range(ticks + 1):
        t = end * i / ticks
        xx = left + t * scale
        yy = top + ranks * lane
        out.append(f'<line x1="{xx:.1f}" y1="{yy}" x2="{xx:.1f}" y2="{yy + 5}" stroke="black"/>')
        out.append(f'<text x="{xx:.1f}" y="{yy + 18}" text-anchor="middle">{t:.1f}</text>')
    out.append(f'<text x="{width / 2:.0f}" y="{top + ranks * lane + 34}" text-anchor="middle">'
               f'ms (simulated step {end:.2f} ms with the optimizer; filled = forward, light = backward)'
               f'</text>')
    out.append("</svg>")
    with open(path, "w") as f:
        f.write("\n".join(out))
    return path
