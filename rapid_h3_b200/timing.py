"""Per-phase timing of the quantized step (the reference's RAPIDH3_TIMING idea, custom_nodes/rapid_h3/__init__.py:
258-264, 817-834: CUDA events around the phases of a fused block, summed when the step is over).

Set `timing.PHASES = {}` to switch it on: every `with phase(name, work):` then brackets its body with two CUDA
events on the current stream and appends (start, stop, work) under `name`; `work` is the phase's algorithmic
operation or byte count. With `PHASES = None` (the default) a phase costs one comparison. Read the result with
`totals()` after synchronising the stream.
"""
import torch

PHASES = None


class phase:
    def __init__(self, name, work=0):
        self.name, self.work = name, work

    def __enter__(self):
        if PHASES is not None:
            self.ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self.ev[0].record()
        return self

    def __exit__(self, *exc):
        if PHASES is not None:
            self.ev[1].record()
            PHASES.setdefault(self.name, []).append((self.ev[0], self.ev[1], self.work))
        return False


def totals(phases=None):
    """{name: {"ms": total milliseconds, "n": brackets, "work": summed work}} of a PHASES dict."""
    phases = PHASES if phases is None else phases
    return {k: {"ms": sum(a.elapsed_time(b) for a, b, _ in v), "n": len(v), "work": sum(w for _, _, w in v)}
            for k, v in phases.items()}
