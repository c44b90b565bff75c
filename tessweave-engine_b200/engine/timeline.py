"""Device-side timeline of the engine's own kernels.

With ``TESSWEAVE_TIMELINE=1`` in the environment the kernels are compiled with a recorder: every
block writes its kernel, its index and three readings of the GPU's global timer (start, after its
wait for the kernel before it, end) into one buffer.  ``Timeline`` owns that buffer; ``launches()``
groups the blocks of a recording into kernel launches, in time order, with for each launch

    start        first block's start (us, from the first launch's start)
    ramp         time until its last block has started
    waited       median time its blocks spent waiting for the kernel before
    first_end    when its first block finished
    end          when its last block finished
    gap          its start minus the end of the launch before (negative: they overlapped)

which is what a step's time is made of when its kernels are short: tails in which few blocks run,
and the dead time between one kernel's end and the next one's first instruction.  Library kernels
(cuBLAS) are not recorded.  The recorder costs an atomic and five stores per block; timings taken
with it are for looking at, not for reporting.
"""
from __future__ import annotations

import torch

from ..csrc import build

KERNEL_NAMES = {1: "embed", 2: "norm", 3: "norm (cluster)", 4: "rope + cache write", 5: "gemm_smallm", 6: "attn_decode",
                7: "attn_prefill", 8: "sample", 9: "silu_mul", 10: "reduce_partial", 11: "other"}
ENTRY_WORDS = 5


class Timeline:
    def __init__(self, capacity: int = 1 << 18, device: str = "cuda"):
        if not build.timeline_enabled():
            raise RuntimeError("the timeline needs TESSWEAVE_TIMELINE=1 in the environment before the first kernel is loaded")
        self.capacity = capacity
        self.buffer = torch.zeros(2 + ENTRY_WORDS * capacity, dtype=torch.int64, device=device)
        self.buffer[1] = capacity
        torch.cuda.synchronize()
        build.set_timeline_buffer(self.buffer.data_ptr())

    def reset(self) -> None:
        """Forget what was recorded (call between steps, with the device idle)."""
        torch.cuda.synchronize()
        self.buffer[0] = 0
        torch.cuda.synchronize()

    def close(self) -> None:
        torch.cuda.synchronize()
        build.set_timeline_buffer(0)

    def entries(self) -> torch.Tensor:
        """[n, 5] int64 on the host: kernel id | blocks << 16, block index, start, after the wait, end (ns)."""
        torch.cuda.synchronize()
        host = self.buffer.cpu()
        n = min(int(host[0]), self.capacity)
        return host[2:2 + ENTRY_WORDS * n].reshape(n, ENTRY_WORDS)

    def launches(self) -> list[dict]:
        return group_launches(self.entries())


def group_launches(entries: torch.Tensor) -> list[dict]:
    """Blocks -> launches.  The blocks of one launch share (kernel, grid size); a launch is complete when as
    many blocks as its grid has have been seen, so two launches of one kernel in a row are told apart."""
    if entries.numel() == 0:
        return []
    order = torch.argsort(entries[:, 2], stable=True)
    rows = entries[order].tolist()
    open_: dict[int, dict] = {}
    done: list[dict] = []
    for tag, _block, t0, t1, t2 in rows:
        cur = open_.get(tag)
        if cur is None:
            cur = open_[tag] = {"kernel": KERNEL_NAMES.get(tag & 0xFFFF, str(tag & 0xFFFF)), "blocks": tag >> 16,
                                "starts": [], "waits": [], "ends": []}
        cur["starts"].append(t0)
        cur["waits"].append(max(0, t1 - t0) if t1 else 0)
        cur["ends"].append(t2)
        if len(cur["starts"]) == cur["blocks"]:
            done.append(open_.pop(tag))
    done.extend(open_.values())               # launches whose blocks were not all recorded
    done.sort(key=lambda c: min(c["starts"]))
    origin = min(done[0]["starts"])
    out: list[dict] = []
    prev_end = None
    for c in done:
        starts, ends = sorted(c["starts"]), sorted(c["ends"])
        waits = sorted(c["waits"])
        row = {"kernel": c["kernel"], "blocks": c["blocks"], "seen": len(starts),
               "start": (starts[0] - origin) / 1e3, "ramp": (starts[-1] - starts[0]) / 1e3,
               "waited": waits[len(waits) // 2] / 1e3, "first_end": (ends[0] - origin) / 1e3,
               "end": (ends[-1] - origin) / 1e3}
        row["gap"] = None if prev_end is None else row["start"] - prev_end
        prev_end = row["end"] if prev_end is None else max(prev_end, row["end"])
        out.append(row)
    return out


def format_launches(rows: list[dict]) -> str:
    head = f"{'kernel':20s} {'blocks':>6s} {'start':>9s} {'gap':>7s} {'ramp':>6s} {'waited':>7s} {'first end':>9s} {'end':>9s} {'length':>7s}"
    lines = [head, "-" * len(head)]
    for r in rows:
        gap = "" if r["gap"] is None else f"{r['gap']:7.2f}"
        lines.append(f"{r['kernel']:20s} {r['blocks']:6d} {r['start']:9.2f} {gap:>7s} {r['ramp']:6.2f} {r['waited']:7.2f} "
                     f"{r['first_end']:9.2f} {r['end']:9.2f} {r['end'] - r['start']:7.2f}")
    return "\n".join(lines)
