"""Generates the committed fixtures under tests/golden/.

ref_expert.npz: outputs of the REFERENCE's own src/backends/cuda/moe_cpu_expert.c (compiled in
place into oracle/_ref by oracle/Makefile) on the reference micro-benches' input distribution
(tools/moe_cpu_bench/moe_exact_bench.cu:102-108): int8 activation codes/scales from
sp_moe_cpu_quant, gate_up and down rows from sp_moe_cpu_gemv. Needs the reference tree and a
CPU with AVX-512 VNNI; run in the build container:  python tests/golden/make_golden.py

layer_*.npz: whole-layer outputs of the checker (oracle/sp_moe_oracle.c) at two small
geometries and both arithmetic flavours; they freeze the checker's behaviour.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import orc  # noqa: E402
from test_oracle_cpu import _bench_inputs  # noqa: E402


def main():
    orc.build_oracle(with_ref=True)
    R = orc.ref_lib()
    if R is None:
        raise SystemExit("oracle/_ref is unavailable here (needs the reference tree and AVX-512 VNNI)")
    seed, E, FFE = 1234, 2816, 704
    gc, gs, dc, ds, x = _bench_inputs(seed)
    qx, sx = np.empty(E, np.int8), np.empty(E // 16, np.float32)
    R.sp_moe_cpu_quant(orc.p(x, orc.f32p), E, orc.p(qx, orc.i8p), orc.p(sx, orc.f32p))
    gu = np.empty(2 * FFE, np.float32)
    R.sp_moe_cpu_gemv(orc.p(gc, orc.u8p), orc.p(gs, orc.u16p), E, 2 * FFE, orc.p(qx, orc.i8p), orc.p(sx, orc.f32p), orc.p(gu, orc.f32p))
    h = (np.random.default_rng(seed + 1).standard_normal(FFE) * 0.05).astype(np.float32)
    hq, hs = np.empty(FFE, np.int8), np.empty(FFE // 16, np.float32)
    R.sp_moe_cpu_quant(orc.p(h, orc.f32p), FFE, orc.p(hq, orc.i8p), orc.p(hs, orc.f32p))
    down = np.empty(E, np.float32)
    R.sp_moe_cpu_gemv(orc.p(dc, orc.u8p), orc.p(ds, orc.u16p), FFE, E, orc.p(hq, orc.i8p), orc.p(hs, orc.f32p), orc.p(down, orc.f32p))
    np.savez_compressed(os.path.join(HERE, "ref_expert.npz"), seed=seed, qx=qx, sx=sx, gate_up=gu, hq=hq, hs=hs, down=down)

    for name, cfg in (("tiny", orc.TINY), ("small", orc.SMALL)):
        for fl, tag in ((0, "A"), (1, "B")):
            seed = 42
            w = orc.make_layer(cfg, seed, rand_norms=True)
            x = np.random.default_rng(seed + 1).standard_normal((5, cfg["E"])).astype(np.float32)
            r = orc.layer_forward(cfg, w, x, fl, True)
            meta = json.dumps(dict(cfg=cfg, seed=seed, flavour=fl))
            np.savez_compressed(os.path.join(HERE, f"layer_{name}_{tag}.npz"), meta=meta, x=x, y=r["y"], sel=r["sel"], wts=r["wts"])
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
