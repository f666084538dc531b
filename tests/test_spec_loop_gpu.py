"""Draft -> verify -> accept on the attention path (crucible_strix_halo_b200/speculative.py): the draft layer is a QSA
layer on its own cache, verify spans commit one row and leave the accepted rows pending, the next pass replays them.
The emitted tokens and the stream's state must equal plain one-row decoding of the same tokens
(engine/engine.hip:444-525; engine/runtime/batch_spec_forward.h:53-130, :159-253; engine/runtime/spec_span.h:6-9)."""
import numpy as np
import pytest
import torch

from tests.gpu_util import rel_l2

pytestmark = pytest.mark.gpu
V = 32


class Glue:
    """Stands in for everything outside the attention core: seeded embedding tables per layer, a little of the layer
    below mixed in (so that a wrong GDN state changes the tokens), a linear head.  Drafts follow a given continuation
    except at chosen positions, which makes acceptance lengths vary."""

    def __init__(self, g, seed):
        gen = torch.Generator(device="cuda").manual_seed(seed)
        rn = lambda *s, std=1.0: torch.randn(*s, device="cuda", generator=gen) * std
        Hv, Hq, C = g.gdn_vheads, g.q_heads, g.gdn_channels
        self.g = g
        self.e_gdn = [(rn(V, C), rn(V, Hv * 128), rn(V, g.hidden)) for _ in range(2)]
        self.m_gdn = rn(Hv * 128, C, std=0.05)
        self.e_qsa = (rn(V, Hq, 512), rn(V, 512), rn(V, 512), rn(V, 640))
        self.m_qsa = rn(Hv * 128, Hq * 512, std=0.05)
        self.e_mtp = (rn(V, Hq, 512), rn(V, 512), rn(V, 512), rn(V, 640))
        self.m_mtp = rn(Hq * 256, 512, std=0.05)
        self.head = rn(Hq * 256, V)
        self.truth, self.wrong = None, set()

    def _t(self, tokens):
        return torch.tensor(tokens, device="cuda", dtype=torch.long)

    def gdn_rows(self, layer, tokens, below):
        t = self._t(tokens)
        qkv, z, x = (e[t].clone() for e in self.e_gdn[layer])
        if below is not None:
            qkv = qkv + below.float() @ self.m_gdn
        return qkv.contiguous(), z.contiguous(), x.contiguous()

    def qsa_rows(self, tokens, below):
        t = self._t(tokens)
        q, k, v, idx = (e[t].clone() for e in self.e_qsa)
        q = q + (below.float() @ self.m_qsa).view(len(tokens), -1, 512)
        return q.contiguous(), k.contiguous(), v.contiguous(), idx.contiguous()

    def mtp_rows(self, tokens, stacks):
        t = self._t(tokens)
        q, k, v, idx = (e[t].clone() for e in self.e_mtp)
        k = k + stacks.float() @ self.m_mtp
        return q.contiguous(), k.contiguous(), v.contiguous(), idx.contiguous()

    def choose(self, out):
        return (out.float() @ self.head).argmax(-1).tolist()

    def draft(self, mtp_out, position):
        if self.truth is not None and position < len(self.truth):
            tok = self.truth[position]
            return (tok + 1) % V if position in self.wrong else tok
        return int((mtp_out.float() @ self.head).argmax())


def _streams(seed, ctx, mtp_rows=0, span=9):
    from crucible_strix_halo_b200 import capi, layers, speculative
    g = capi.Geometry(256, 16, 2, 4, 2)
    rng = np.random.default_rng(seed)
    gw = [layers.GdnWeights(g, 0.5 * rng.normal(size=(g.gdn_channels, 4)), rng.normal(size=4) - 1, 0.5 * rng.normal(size=4),
                            1 + 0.1 * rng.normal(size=128), ab=0.05 * rng.normal(size=(8, 256))) for _ in range(2)]
    qw, mw = (layers.QsaWeights(g, *[1 + 0.1 * rng.normal(size=n) for n in (256, 256, 128, 128)]) for _ in range(2))
    glue = Glue(g, seed)
    make = lambda: speculative.SpecStream(g, gw, qw, mw, glue, ctx, mtp_rows=mtp_rows, span=span)
    return capi, glue, make


@pytest.mark.parametrize("span", [9, 5])
def test_speculative_rounds_equal_plain_decoding(span):
    capi, glue, make = _streams(21 + span, ctx=256, span=span)
    prompt = [3, 17, 4, 9, 30, 1]
    total = 120
    # plain greedy decoding, one row per step: the continuation every draft is judged against
    plain = make()
    plain.feed(prompt)
    while len(plain.tokens) < total:
        plain.decode_one()
    truth = list(plain.tokens)
    # drafts follow the continuation except at seeded positions, so passes accept 0 .. span - 1 rows
    glue.truth = truth
    rng = np.random.default_rng(5)
    glue.wrong = set(int(p) for p in rng.choice(np.arange(len(prompt), total), size=total // 5, replace=False))
    spec = make()
    spec.feed(prompt)
    while len(spec.tokens) < total - span:
        spec.round()
    assert spec.tokens == truth[:len(spec.tokens)], "speculative decoding changed the tokens"
    assert min(spec.accepted) == 0 and max(spec.accepted) == span - 1 and len(set(spec.accepted)) >= 3, spec.accepted
    # the same tokens, plainly decoded, leave the same state
    ref = make()
    glue.truth = None
    ref.feed(truth[:len(spec.tokens)])
    a, b = spec.flush(), ref.flush()
    assert (a - b).abs().max().item() < 1e-4
    L = len(spec.tokens)
    for s, r in zip(spec.gs, ref.gs):
        assert rel_l2(s.state_view().cpu().numpy(), r.state_view().cpu().numpy()) < 1e-5
        keep = [p & 15 for p in range(L - 3, L)]      # the conv taps of the next row; older slots may hold rejected draft rows
        assert (s.hist[keep] - r.hist[keep]).abs().max().item() < 1e-4          # rows of the layer below differ in the last bits
    assert (spec.qs.k[:L].float() - ref.qs.k[:L].float()).abs().max().item() < 2e-3
    assert (spec.qs.v[:L].float() - ref.qs.v[:L].float()).abs().max().item() < 2e-3
    nb = L // 4
    assert (spec.qs.pool_rows(nb) - ref.qs.pool_rows(nb)).abs().max().item() < 1e-4      # no pooled key kept a rejected row
    # the draft layer's cache: rows below mpos were rewritten from the trunk's own outputs (catch-up rows)
    ref._draft(1)
    m = min(spec.mpos, ref.mpos)
    assert m >= L - span - 1
    assert (spec.ms.k[:m].float() - ref.ms.k[:m].float()).abs().max().item() < 2e-3
    assert (spec.ms.v[:m].float() - ref.ms.v[:m].float()).abs().max().item() < 2e-3


def test_draft_layer_cache_is_bounded():
    capi, glue, make = _streams(4, ctx=64, mtp_rows=12, span=5)
    s = make()
    s.feed([1, 2, 3, 4, 5, 6, 7, 8])
    s.round()
    with pytest.raises(ValueError):
        while True:
            s.round()
