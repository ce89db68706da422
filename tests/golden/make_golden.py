"""Generate the golden fixtures by executing the reference's own source files.

Run where the reference checkout is readable:

    python tests/golden/make_golden.py --reference /path/to/tensor-product-attention-jax [--only bwd]

jax is not installed there, so the reference files (tpa/tpa.py, tpa/mha.py,
tpa/ring_tpa.py, tpa/tpa_test.py) are imported unmodified on top of the numpy
stand-in in _jax_standin.py.  Inputs come from oracle.make_factors (numpy
Philox, seed stored with each case), because jax.random is not available; the
tests regenerate them from the stored seed and compare against the stored
outputs.  The script also re-runs the reference's own assertion (Pallas kernel
vs its test-file reference(), rtol = atol = 1e-3) on every forward case.

Writes tests/golden/fwd_matrix.npz, ring_matrix.npz, extra.npz, bwd_matrix.npz.
"""

from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from oracle.tpa_oracle import make_factors, segment_ids  # noqa: E402

# tpa/tpa_test.py:63-73
FWD_SHAPES = [
    (1, 8, 8, 1, 4, 6, 8),
    (2, 1024, 128, 2, 3, 5, 42),
    (2, 1024, 128, 2, 3, 5, None),
    (2, 128, 1024, 2, 3, 5, 42),
    (2, 128, 1024, 2, 3, 5, None),
    (1, 1024, 1024, 2, 3, 5, 321),
]
# tpa/ring_tpa_test.py:63-70
RING_SHAPES = [
    (1, 16, 16, 1, 4, 6),
    (2, 1024, 128, 4, 32, 8),
    (2, 128, 1024, 4, 32, 8),
]
RANKS_Q = [1, 6]
RANKS_K = [1, 4]


def load_reference(ref_root):
    """Import the reference files under the module names their own imports expect."""
    import _jax_standin

    _jax_standin.install()

    def load(name, path):
        spec = importlib.util.spec_from_file_location(name, path)
        m = importlib.util.module_from_spec(spec)
        sys.modules[name] = m
        spec.loader.exec_module(m)
        return m

    def pkg(name):
        m = types.ModuleType(name)
        m.__path__ = []
        sys.modules[name] = m
        return m

    tdir = os.path.join(ref_root, "tpa")
    # tpa/tpa_test.py:15-16 imports models.attention.kernels.tpa and models.attention.mha
    models, att, kern = pkg("models"), pkg("models.attention"), pkg("models.attention.kernels")
    models.attention, att.kernels = att, kern
    tpa = load("models.attention.kernels.tpa", os.path.join(tdir, "tpa.py"))
    kern.tpa = tpa
    mha = load("models.attention.mha", os.path.join(tdir, "mha.py"))
    att.mha = mha
    # tpa/ring_tpa.py:21 does `from .kernels import tpa`
    rpkg = pkg("refpkg")
    rk = pkg("refpkg.kernels")
    rk.tpa = tpa
    rpkg.kernels = rk
    ring = load("refpkg.ring_tpa", os.path.join(tdir, "ring_tpa.py"))
    ttest = load("ref_tpa_test", os.path.join(tdir, "tpa_test.py"))
    return tpa, mha, ring, ttest


def make_backward(tpa, ttest):
    """Backward matrix of tpa/tpa_test.py:128-140: the reference's own _tpa_bwd (materialising
    branch; the nomat branch needs jax's functional `.at[].add`, which numpy arrays lack) on the
    residuals of its own forward, non-causal as in the reference's test, for a random `do`."""
    bw = {}
    seed = 300
    for shape in FWD_SHAPES:
        b, lq, lk, h, dk, dv, seg = shape
        for rq in RANKS_Q:
            for rk in RANKS_K:
                seed += 1
                q, k, v = make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist="normal")
                do = np.random.Generator(np.random.Philox(key=seed + 5000)).standard_normal(
                    (b, lq, h, dv), dtype=np.float32)
                qs = segment_ids(b, lq, seg) if seg else None
                ks = segment_ids(b, lk, seg) if seg else None
                _, res = tpa._tpa_fwd(
                    q, k, v, num_heads=h, q_segment_ids=qs, kv_segment_ids=ks, sm_scale=1.0,
                    causal=False, block_sizes=None, nomat=False, debug=False, interpret=True,
                )
                dq, dk_, dv_, _, _ = tpa._tpa_bwd(h, 1.0, False, None, False, False, True, res, do)
                key = f"b{b}_lq{lq}_lk{lk}_h{h}_dk{dk}_dv{dv}_seg{seg or 0}_rq{rq}_rk{rk}"
                bw[key + "/meta"] = np.array([seed, b, lq, lk, rq, rk, h, dk, dv, seg or 0])
                bw[key + "/dq"] = np.asarray(dq, np.float32)
                bw[key + "/dk"] = np.asarray(dk_, np.float32)
                bw[key + "/dv"] = np.asarray(dv_, np.float32)
    print(f"backward matrix: {len(bw) // 4} cases")
    np.savez_compressed(os.path.join(HERE, "bwd_matrix.npz"), **bw)
    print("bwd_matrix.npz", os.path.getsize(os.path.join(HERE, "bwd_matrix.npz")) // 1024, "KiB")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TPA_REFERENCE"), required="TPA_REFERENCE" not in os.environ,
                    help="checkout of jondeaton/tensor-product-attention-jax (or set TPA_REFERENCE)")
    ap.add_argument("--only", choices=["all", "bwd"], default="all",
                    help="bwd: regenerate bwd_matrix.npz only")
    args = ap.parse_args()
    tpa, mha, ring, ttest = load_reference(args.reference)
    import _jax_standin as js

    make_backward(tpa, ttest)
    if args.only == "bwd":
        return

    # ---------------------------------------------------------------- forward matrix
    fwd = {}
    seed = 100
    worst = 0.0
    for shape in FWD_SHAPES:
        b, lq, lk, h, dk, dv, seg = shape
        for rq in RANKS_Q:
            for rk in RANKS_K:
                seed += 1
                q, k, v = make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist="uniform")
                qs = segment_ids(b, lq, seg) if seg else None
                ks = segment_ids(b, lk, seg) if seg else None
                ref = ttest.reference(q, k, v, q_segment_ids=qs, kv_segment_ids=ks, num_heads=h)
                outs = {}
                for nomat in (False, True):
                    o, res = tpa._tpa_fwd(
                        q, k, v, num_heads=h, q_segment_ids=qs, kv_segment_ids=ks, sm_scale=1.0,
                        causal=False, block_sizes=None, nomat=nomat, debug=False, interpret=True,
                    )
                    np.testing.assert_allclose(o, ref, rtol=1e-3, atol=1e-3)  # tpa/tpa_test.py:125
                    outs[nomat] = (o, res[-1])
                worst = max(worst, float(np.max(np.abs(outs[False][0] - ref))))
                worst = max(worst, float(np.max(np.abs(outs[True][0] - outs[False][0]))))
                key = f"b{b}_lq{lq}_lk{lk}_h{h}_dk{dk}_dv{dv}_seg{seg or 0}_rq{rq}_rk{rk}"
                fwd[key + "/meta"] = np.array([seed, b, lq, lk, rq, rk, h, dk, dv, seg or 0])
                fwd[key + "/o"] = outs[False][0].astype(np.float32)
                fwd[key + "/lse"] = outs[False][1].astype(np.float32)
    print(f"forward matrix: {len(fwd) // 3} cases, kernel vs reference()/nomat max-abs {worst:.3e}")
    np.savez_compressed(os.path.join(HERE, "fwd_matrix.npz"), **fwd)

    # ---------------------------------------------------------------- ring matrix (8 shards, segment size 42)
    rg = {}
    worst = 0.0
    for shape in RING_SHAPES:
        b, lq, lk, h, dk, dv = shape
        for rq in RANKS_Q:
            for rk in RANKS_K:
                seed += 1
                q, k, v = make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist="uniform")
                qs, ks = segment_ids(b, lq, 42), segment_ids(b, lk, 42)
                ref = ttest.reference(q, k, v, q_segment_ids=qs, kv_segment_ids=ks, num_heads=h)

                def per_shard(q, k, v, qs, ks, h=h):
                    return ring.ring_tpa(q, k, v, qs, ks, axis_name="sp", num_heads=h,
                                         debug=False, interpret=True)

                o = js.run_sharded(per_shard, 8, [q, k, v, qs, ks])
                np.testing.assert_allclose(o, ref, rtol=1e-3, atol=1e-3)  # tpa/ring_tpa_test.py:138
                worst = max(worst, float(np.max(np.abs(o - ref))))
                key = f"b{b}_lq{lq}_lk{lk}_h{h}_dk{dk}_dv{dv}_rq{rq}_rk{rk}"
                rg[key + "/meta"] = np.array([seed, b, lq, lk, rq, rk, h, dk, dv, 42, 8])
                rg[key + "/o"] = o.astype(np.float32)
    print(f"ring matrix: {len(rg) // 2} cases, ring vs reference() max-abs {worst:.3e}")
    np.savez_compressed(os.path.join(HERE, "ring_matrix.npz"), **rg)

    # ---------------------------------------------------------------- behaviour the reference's tests never execute
    ex = {}

    def fwd_case(name, seed, b, lq, lk, rq, rk, h, dk, dv, seg_q, seg_k, sm_scale, causal, dist):
        q, k, v = make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist=dist)
        qs = segment_ids(b, lq, seg_q) if seg_q else None
        ks = segment_ids(b, lk, seg_k) if seg_k else None
        o, res = tpa._tpa_fwd(
            q, k, v, num_heads=h, q_segment_ids=qs, kv_segment_ids=ks, sm_scale=sm_scale,
            causal=causal, block_sizes=None, nomat=False, debug=False, interpret=True,
        )
        with np.errstate(invalid="ignore"):
            ref = ttest.reference(q, k, v, q_segment_ids=qs, kv_segment_ids=ks, num_heads=h,
                                  sm_scale=sm_scale, causal=causal)
        np.testing.assert_allclose(o, ref, rtol=1e-3, atol=1e-3, equal_nan=True)
        ex[name + "/meta"] = np.array(
            [seed, b, lq, lk, rq, rk, h, dk, dv, seg_q or 0, seg_k or 0, int(causal),
             {"normal": 0, "uniform": 1}[dist]]
        )
        ex[name + "/sm_scale"] = np.array(sm_scale, dtype=np.float64)
        ex[name + "/o"] = o.astype(np.float32)
        ex[name + "/lse"] = res[-1].astype(np.float32)
        print(f"{name}: nan rows {int(np.isnan(o).any(-1).sum())}, max-abs vs reference() "
              f"{float(np.nanmax(np.abs(o - ref))):.3e}")

    # configuration 0 of the benchmark: fp32 causal B1 T512 h8 d64 R 6/2/2, sm_scale 1/sqrt(d)
    fwd_case("c0_causal", 0, 1, 512, 512, 6, 2, 8, 64, 64, None, None, 64**-0.5, True, "normal")
    fwd_case("causal_seg", 7, 2, 256, 256, 3, 2, 2, 8, 8, 42, 42, 0.3, True, "normal")
    fwd_case("peaky", 8, 1, 256, 256, 2, 2, 4, 16, 16, None, None, 6.0, True, "normal")
    # query segments 4.. have no key with the same id -> empty rows -> NaN (tpa/tpa.py:439)
    fwd_case("empty_rows", 9, 1, 256, 128, 2, 2, 2, 8, 8, 42, 42, 1.0, False, "uniform")

    def ring_case(name, seed, n, b, l, rq, rk, h, dk, dv, seg, sm_scale, causal):
        q, k, v = make_factors(seed, b, l, l, rq, rk, h, dk, dv, dist="normal")
        qs = segment_ids(b, l, seg) if seg else np.zeros((b, l), np.int32)
        ks = qs.copy()

        def per_shard(q, k, v, qs, ks):
            return ring.ring_tpa(q, k, v, qs, ks, axis_name="sp", num_heads=h, sm_scale=sm_scale,
                                 causal=causal, debug=False, interpret=True)

        o = js.run_sharded(per_shard, n, [q, k, v, qs, ks])
        ex[name + "/meta"] = np.array([seed, b, l, l, rq, rk, h, dk, dv, seg or 0, n, int(causal)])
        ex[name + "/sm_scale"] = np.array(sm_scale, dtype=np.float64)
        ex[name + "/o"] = o.astype(np.float32)
        print(f"{name}: shape {o.shape}, nan {int(np.isnan(o).sum())}")

    # ring with causal=True: the reference masks on shard-local indices at every step
    ring_case("ring_causal_n4", 10, 4, 1, 512, 2, 2, 4, 16, 16, None, 0.25, True)
    ring_case("ring_causal_n8_seg", 11, 8, 1, 1024, 3, 2, 2, 8, 8, 100, 0.35, True)
    np.savez_compressed(os.path.join(HERE, "extra.npz"), **ex)
    for f in ("fwd_matrix.npz", "ring_matrix.npz", "extra.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    main()
