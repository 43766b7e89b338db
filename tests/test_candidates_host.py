"""The arbiter seam without a GPU: registry, tier priority, forcing, measuring, and which
regions each sm_100a candidate accepts (python/tessera/compiler/emit/candidate.py:110-236)."""
import pytest

from tessera_b200 import candidates as cd


class _Fake(cd.Candidate):
    target = "nvidia"
    op = cd.OP_MATMUL

    def __init__(self, name, tier, ok=True, applies=True):
        self.name, self.tier, self._ok, self._applies = name, tier, ok, applies

    def available(self):
        return self._ok

    def applies_to(self, region):
        return self._applies

    def run(self, region, *inputs, **kw):
        return self.name, "fake_kernel"


@pytest.fixture(autouse=True)
def _clean():
    cd._CANDIDATES.clear()
    yield
    cd._CANDIDATES.clear()


def test_registry_and_arbiter():
    lo, hi = _Fake("emitted", cd.Tier.EMITTED), _Fake("hand", cd.Tier.HAND_TUNED)
    gone = _Fake("offline", cd.Tier.HAND_TUNED, ok=False)
    cd.register_candidate(lo)
    cd.register_candidate(hi)
    cd.register_candidate(gone)
    assert [c.name for c in cd.candidates_for("nvidia", cd.OP_MATMUL)] == ["emitted", "hand", "offline"]
    r = cd.MatmulRegion()
    assert cd.arbitrate("nvidia", cd.OP_MATMUL, r) is hi                       # highest tier wins
    assert cd.arbitrate("nvidia", cd.OP_MATMUL, r, force="emitted") is lo      # escape hatch
    assert cd.arbitrate("nvidia", cd.OP_MATMUL, r, measure=lambda c: 1.0 if c is hi else 0.5) is lo
    with pytest.raises(cd.ArbiterError):
        cd.arbitrate("nvidia", cd.OP_MATMUL, r, force="offline")
    with pytest.raises(cd.ArbiterError):
        cd.arbitrate("nvidia", cd.OP_ATTENTION, r)
    assert cd.run_arbitrated("nvidia", cd.OP_MATMUL, r) == ("hand", "fake_kernel", "hand")
    cd.register_candidate(_Fake("hand", cd.Tier.SYNTHESIZED))                  # same name replaces
    assert len(cd.candidates_for("nvidia", cd.OP_MATMUL)) == 3
    assert cd.arbitrate("nvidia", cd.OP_MATMUL, r) is lo
    with pytest.raises(ValueError):
        cd.register_candidate(_Fake("", cd.Tier.EMITTED))
    bad = _Fake("x", cd.Tier.EMITTED)
    bad.op = "nonsense"
    with pytest.raises(ValueError):
        cd.register_candidate(bad)


def test_which_regions_the_sm100_candidates_accept():
    fused = cd.Sm100FusedGemm()
    ok = [cd.FusedRegion(()), cd.FusedRegion(("bias",)), cd.FusedRegion(("bias", "gelu")), cd.FusedRegion(("silu",)),
          cd.FusedRegion(("bias",), residual=True), cd.FusedRegion((), residual=True, storage_dtype="f16")]
    no = [cd.FusedRegion(("gelu", "bias")), cd.FusedRegion(("relu", "silu")), cd.FusedRegion(("tanh",)),
          cd.FusedRegion(("bias", "relu"), residual=True), cd.FusedRegion((), reduction="softmax"),
          cd.FusedRegion((), prologue=("gelu",)), cd.FusedRegion((), storage_dtype="fp8_e4m3")]
    assert all(fused.applies_to(r) for r in ok)
    assert not any(fused.applies_to(r) for r in no)
    gated = cd.Sm100GatedMatmul()
    assert gated.applies_to(cd.GatedMatmulRegion("silu")) and not gated.applies_to(cd.GatedMatmulRegion("gelu"))
    att = cd.Sm100Attention()
    assert att.applies_to(cd.AttentionRegion()) and not att.applies_to(cd.AttentionRegion(storage_dtype="f16"))
    cs = cd.register_sm100_candidates()
    assert {c.op for c in cs} == {cd.OP_MATMUL, cd.OP_FUSED_REGION, cd.OP_ATTENTION, cd.OP_GATED_MATMUL}
    assert all(c.tier is cd.Tier.HAND_TUNED and c.target == "nvidia" for c in cs)
