"""Where the time of a decode step goes: %globaltimer stamps from a measurement build of the library.

Build a second copy of the library with the stamps compiled in and point this module at it:

    EXL3_B200_BUILD_OUT=/tmp/libexl3_timeline.so EXL3_B200_BUILD_OBJ=/tmp/exl3_timeline_obj EXL3_B200_NVCC_FLAGS=-DEXL3_TIMELINE \\
        python -m trellis_serve_b200.csrc.build
    python -m trellis_serve_b200.runtime.step_timeline --lib /tmp/libexl3_timeline.so --layers 8

In that build thread 0 of every CTA of the decode GEMV and of the attention kernel writes the time at a few points
(kernel entry, dependency wait resolved, own input rotated, first weights landed, loop end, kernel end; attention: scores,
values, hand-over count, merge end).  The report gives, per linear of a layer, those points relative to the end of the GEMV
launch ahead of it (median over layers), i.e. what sits on the critical path between two linears.  The stamps cost a few
stores per CTA; the normal build has none of this code.
"""
from __future__ import annotations

import argparse
import ctypes

import numpy as np
import torch

TL_POINTS, TL_SLOTS, TL_CTAS = 12, 128, 512


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--lib", required=True, help="library built with -DEXL3_TIMELINE")
    ap.add_argument("--layers", type=int, default=8, help="layers of the 27B shape (4 GEMV launches each; at most 32 fit the stamp buffer)")
    ap.add_argument("--context", type=int, default=2048)
    args = ap.parse_args()
    from .. import _lib
    _lib.LIB_PATH = args.lib
    from .decode_step import DecodeStep, ModelShape
    lib = _lib.load()
    lib.exl3_debug_timeline.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
    lib.exl3_debug_att_timeline.argtypes = [ctypes.c_void_p]
    dev = torch.device("cuda:0")
    layers = min(args.layers, TL_SLOTS // 4)
    st = DecodeStep(ModelShape(layers=layers), 3, 0, args.context, device=dev)
    st.h_in.normal_()
    st.capture()
    for _ in range(3):
        st.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    st.replay()
    e1.record()
    torch.cuda.synchronize()
    print(f"step of {layers} layers: {e0.elapsed_time(e1) * 1e3 / layers:.1f} us per layer")
    buf = np.zeros((TL_SLOTS, TL_CTAS, TL_POINTS), dtype=np.uint64)
    nxt = ctypes.c_int(0)
    assert lib.exl3_debug_timeline(buf.ctypes.data, ctypes.byref(nxt)) == 0
    t = buf.astype(np.int64)
    big = np.iinfo(np.int64).max
    first = np.where(t[:, :, 0] > 0, t[:, :, 0], big).min(axis=1)
    order = [i for i in np.argsort(first) if first[i] < big][-layers * 4:]           # the GEMV launches of the last replay, in time order
    t = t[order]
    n = len(order)
    names = ["qkv", "o", "gate_up", "down"]
    rows = {k: [] for k in names}

    def grid_of(i):
        return int((t[i, :, 0] > 0).sum())

    for i in range(4, n):
        a, prev = t[i, :grid_of(i)], t[i - 1, :grid_of(i - 1)]
        prev_end = prev[:, 5].max()

        def rel(p, f):
            v = a[:, p]
            v = v[v > 0]
            return f(v) - prev_end if len(v) else float("nan")
        rows[names[i % 4]].append([rel(0, np.min), rel(0, np.max), rel(1, np.min), rel(1, np.max), rel(2, np.median), rel(3, np.median),
                                   rel(3, np.max), rel(4, np.median), rel(4, np.max), rel(5, np.max)])
    hdr = ["entry.min", "entry.max", "wait.min", "wait.max", "rotated.med", "stage0.med", "stage0.max", "loopend.med", "loopend.max", "end.max"]
    print("decode GEMV, ns after the end of the GEMV launch ahead (median over layers); end.max is the launch's period:")
    for k in names:
        if rows[k]:
            r = np.median(np.array(rows[k], dtype=np.float64), axis=0)
            print(f"  {k:8s} " + "  ".join(f"{h}={v:.0f}" for h, v in zip(hdr, r)))
    ab = np.zeros((64, 256, 8), dtype=np.uint64)
    assert lib.exl3_debug_att_timeline(ab.ctypes.data) == 0
    ab = ab.astype(np.int64)
    qkv_ends = sorted(int(t[i, :grid_of(i), 5].max()) for i in range(n) if i % 4 == 0)
    o_waits = sorted(int(t[i, :grid_of(i), 1].min()) for i in range(n) if i % 4 == 1)
    res = []
    for sl in range(64):                          # attention slots are keyed by the cache address: one per layer
        a = ab[sl]
        a = a[a[:, 0] > 0]
        if not len(a):
            continue
        prev = [e for e in qkv_ends if e <= a[:, 1].max()]
        if not prev:
            continue
        base = prev[-1]
        nxt_o = [w for w in o_waits if w >= base]

        def mx(pt):
            v = a[:, pt][a[:, pt] > 0]
            return (v.max() - base) if len(v) else float("nan")
        res.append([a[:, 0].min() - base, a[:, 1].max() - base, np.median(a[:, 2]) - base, mx(2), np.median(a[:, 3]) - base, mx(3), mx(4), mx(5),
                    mx(7), (nxt_o[0] - base) if nxt_o else float("nan")])
    if res:
        hdr2 = ["entry.min", "wait.max", "scores.med", "scores.max", "values.med", "values.max", "count.max", "fence.max", "merge.end", "o.wait"]
        r = np.median(np.array(res, dtype=np.float64), axis=0)
        print("attention, ns after the end of the q|k|v launch ahead (median over layers):")
        print("  " + "  ".join(f"{h}={v:.0f}" for h, v in zip(hdr2, r)))


if __name__ == "__main__":
    main()
