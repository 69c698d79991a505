"""Generates tests/golden/slha_golden.npz with the CPU oracle (run from the repo root:
`python tests/golden/make_golden.py`).  The reference (Rust) cannot be run on the
build machine, so these vectors are the oracle's output on seeded inputs; the
oracle itself is pinned by the reference's known-answer tests.  The fixture holds,
per codec: keys, the projection, the 128-byte tiles, prepared queries, scores and
the top-16 indices, for d = 160 (with and without the Hadamard transform)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import pyoracle as ora  # noqa: E402
from tests import helpers as H  # noqa: E402


def main():
    out = {}
    d, n, nq = 160, 96, 3
    for rht in (0, 1):
        p = H.orthogonal_projection(300 + rht, d)
        model = ora.Model(p, d, seed=40 + rht, rht=bool(rht))
        keys = H.to_bf16_f32(H.gaussian_keys(500 + rht, n, d, outlier_channels=(7, 93)))
        q = H.gaussian_keys(600 + rht, nq, d)
        prep = [model.prepare_query(x) for x in q]
        qc = np.stack([a for a, _ in prep])
        qs = np.stack([b for _, b in prep])
        tag = "rht%d_" % rht
        out[tag + "projection"], out[tag + "keys"], out[tag + "queries"] = p, keys, q
        out[tag + "q_coarse"], out[tag + "q_sign"] = qc, qs
        for codec in range(7):
            tiles = model.encode_batch(keys, codec, pos=np.arange(n, dtype=np.uint32) + 11)
            scores = H.oracle_scores(tiles, qc, qs)
            top = np.stack([ora.topk(scores[j], 16)[0] for j in range(nq)])
            out[tag + "tiles_c%d" % codec] = tiles.view(np.uint8).reshape(n, 128)
            out[tag + "scores_c%d" % codec] = scores
            out[tag + "top16_c%d" % codec] = top
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "slha_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
