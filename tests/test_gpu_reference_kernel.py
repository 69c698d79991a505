"""The reference's own CUDA scoring kernel (slhav2-vram/kernels/slha_score.cu, built into
oracle/_ref/ where the reference tree was mounted) as a second checker: the CPU restatement and the
library must both agree with the reference's real device code on the same tiles."""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32

needs_ref = pytest.mark.skipif(ora.ref_cuda_library() is None,
                               reason="oracle/_ref/libslha_ref_cuda.so was not built (reference tree absent at build time)")


@needs_ref
@pytest.mark.parametrize("codec", [0, 1, 2, 3, 4, 5])
def test_oracle_and_library_match_the_reference_cuda_kernel(codec):
    n, nq = 3000, 3
    tiles = H.random_tiles(n, codec, seed=40 + codec, warm_every=7, nocorr_every=5)
    qc, qs = H.random_queries(nq, 50 + codec)
    ref = ora.ref_cuda_scores(tiles, qc, qs)
    want = H.oracle_scores(tiles, qc, qs)
    got = S.score_tiles(tiles, n, qc, qs, nq)
    tol = 1e-3 * (1 + np.abs(ref))  # the reference's own tolerance (scirust/src/attention/slha_v2/tests.rs:542)
    assert np.all(np.abs(want - ref) <= tol)
    assert np.all(np.abs(got - ref) <= tol)
    assert np.max(np.abs(got - ref)) <= 1e-3


@needs_ref
def test_reference_cuda_kernel_known_answers():
    # slhav2-vram/tests/cpu.rs:53-115: latent 0x88 / 0x00 / 0xFF, scale 1, gs 255, q = 1 -> 0 / -1024 / +896
    tiles = np.zeros(3, S.TILE_DTYPE)
    tiles["scale"] = 1.0
    tiles["group_scales"] = 255
    tiles["flags"] = 1  # WARM: coarse term only
    tiles["latent_kv"][0] = 0x88
    tiles["latent_kv"][1] = 0x00
    tiles["latent_kv"][2] = 0xFF
    qc = np.ones((1, 128), F)
    qs = np.zeros((1, 4), np.uint64)
    ref = ora.ref_cuda_scores(tiles, qc, qs)[0]
    assert np.allclose(ref, [0.0, -1024.0, 896.0], atol=1e-4)
    assert np.allclose(ora.score_tiles(tiles, qc[0], qs[0]), ref, atol=1e-4)
    assert np.allclose(S.score_tiles(tiles, 3, qc, qs, 1)[0], ref, atol=1e-4)
