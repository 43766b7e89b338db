"""The four sm_100a candidates run real kernels and match the region oracles."""
import os

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, no_device_error, rel_err

pytestmark = pytest.mark.gpu

from tessera_b200 import candidates as cd  # noqa: E402
from tessera_b200.device import bfloat16  # noqa: E402


def test_candidates_against_region_oracles(golden_dir):
    g = np.load(os.path.join(golden_dir, "gemm.npz"))
    cd._CANDIDATES.clear()
    cs = cd.register_sm100_candidates()
    assert all(c.available() for c in cs)
    out, tag, name = cd.run_arbitrated("nvidia", cd.OP_MATMUL, cd.MatmulRegion("bfloat16"), g["A0"][0], g["B0"][0])
    assert tag == cd.EXECUTION_TAG and name == "sm100_tcgen05_gemm"
    assert rel_err(out, orc.gemm(g["A0"][0].astype(bfloat16), g["B0"][0].astype(bfloat16))) < 1e-4
    for act in ("linear", "relu", "gelu", "silu"):
        ep = ("bias",) + (() if act == "linear" else (act,))
        out, tag, _ = cd.run_arbitrated("nvidia", cd.OP_FUSED_REGION, cd.FusedRegion(ep), g["epiA"], g["epiB"],
                                        bias=g["epi_bias"])
        ref = orc.fused_epilogue(orc.gemm(g["epiA"], g["epiB"]), bias=g["epi_bias"], activation=act)
        assert tag == cd.EXECUTION_TAG and rel_err(out, ref) < 1e-4
    out, _, _ = cd.run_arbitrated("nvidia", cd.OP_FUSED_REGION, cd.FusedRegion(("bias",), residual=True),
                                  g["epiA"], g["epiB"], bias=g["epi_bias"], residual=g["epi_res"])
    assert rel_err(out, g["epi_linear"]) < 1e-4
    out, tag, _ = cd.run_arbitrated("nvidia", cd.OP_GATED_MATMUL, cd.GatedMatmulRegion("silu"), g["gatedA"],
                                    g["gatedWg"], g["gatedWu"])
    assert tag == cd.EXECUTION_TAG and rel_err(out, g["gatedO"]) < TOL
    sc = float(1.0 / np.sqrt(128.0))
    for causal, key in ((False, "regO"), (True, "regOc")):
        out, tag, _ = cd.run_arbitrated("nvidia", cd.OP_ATTENTION, cd.AttentionRegion(sc, causal), g["regQ"],
                                        g["regK"], g["regV"])
        assert tag == cd.EXECUTION_TAG and rel_err(out, g[key]) < TOL
    with pytest.raises(ValueError):     # top-left causal mask with M != Nk is not what the kernel computes
        cd.Sm100Attention().run(cd.AttentionRegion(sc, True), g["regQ"][:50], g["regK"], g["regV"])
    ms = cd.Sm100Matmul().measure_device_latency(cd.MatmulRegion("bfloat16"), g["epiA"], g["epiB"], reps=5, warmup=2)
    assert ms is not None and 0 < ms < 50
    no_device_error()
    cd._CANDIDATES.clear()
