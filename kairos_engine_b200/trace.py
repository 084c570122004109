"""Expert-route trace in the reference's file format (SP_MOE_TRACE=1 + SP_MOE_TRACE_FILE,
src/backends/cuda/cuda_forward.cu:8546-8593), so its replay/analysis scripts read this path too.

One line per (layer, token):   R <fwd> <P|D> <L> <t> <us> e:w:h,e:w:h,...
  fwd  forward counter (bumped once per call), P = batched call, D = single-token decode,
  us   microseconds since the trace was opened, e = expert id in descending probability,
  w    its renormalised gate weight (%.4f), h = 1: resident in device memory (always, here: the
       whole expert set lives in HBM; the reference prints 0/1 for its slot cache, -1 without one).
Without SP_MOE_TRACE_FILE the reference prints "[moe-route] L=<L> t=<t> e=<ids>" to stderr; so does this.
"""
import os
import sys
import time


def format_lines(fwd, sel, wts, layer_first, us):
    """sel, wts: [n_layers][M][NU] (numpy). Returns the trace lines of one forward call."""
    n_layers, M, NU = sel.shape
    phase = "D" if M == 1 else "P"
    out = []
    for li in range(n_layers):
        for t in range(M):
            items = ",".join(f"{int(sel[li, t, k])}:{float(wts[li, t, k]):.4f}:1" for k in range(NU))
            out.append(f"R {fwd} {phase} {layer_first + li} {t} {us} {items}")
    return out


class RouteTrace:
    """Armed by SP_MOE_TRACE=1 (read once, as the reference does); a no-op otherwise."""

    def __init__(self, env=os.environ):
        self.on = env.get("SP_MOE_TRACE", "") [:1] == "1"
        self.path = env.get("SP_MOE_TRACE_FILE") or None
        self.fwd = 0
        self.t0 = time.monotonic()
        self._f = None
        if self.on and self.path:
            self._f = open(self.path, "a", buffering=1 << 20)

    def record(self, sel, wts, layer_first=0):
        if not self.on or sel is None:
            return
        self.fwd += 1
        if self._f is not None:
            us = int((time.monotonic() - self.t0) * 1e6)
            self._f.write("\n".join(format_lines(self.fwd, sel, wts, layer_first, us)) + "\n")
            if sel.shape[1] == 1:
                self._f.flush()
        else:
            for li in range(sel.shape[0]):
                for t in range(sel.shape[1]):
                    print(f"[moe-route] L={layer_first + li} t={t} e=" + ",".join(str(int(e)) for e in sel[li, t]), file=sys.stderr)

    def close(self):
        if self._f is not None:
            self._f.close()
            self._f = None
