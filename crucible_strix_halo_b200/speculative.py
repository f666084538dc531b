"""Draft -> verify -> accept over the attention path, with the draft (MTP) layer reused as one more QSA layer on a
cache of its own.

The reference drafts with its MTP layer, which is a QSA layer at index kLayers with its own cache of `mtp_capacity` rows
(Engine::Mtp / MtpSpans, engine/engine.hip:444-525, engine/runtime/batch_spec_forward.h:53-130), verifies a span of
1 certain + d draft rows through the trunk with commit = 1 (engine/runtime/spec_span.h:6-9), keeps the accepted rows
as pending GDN rows that the next pass replays (engine/layers/ops.h:275-293) and rewrites the draft layer's rows of
the accepted positions from the trunk's outputs ("catch-up" rows of an R-row MTP pass).

Everything outside the attention core (embeddings, projections, heads) is the caller's: a `glue` object turns tokens
and the previous layer's rows into projection rows and output rows into tokens.  This module only orders the calls of
the C ABI and keeps the ledger; it is host logic, every computation happens in libcrucible_attn.so.

glue protocol:
    gdn_rows(layer, tokens, below)   -> (qkv [R,C], z [R,Hv*128], x [R,hidden])       fp32 cuda tensors
    qsa_rows(tokens, below)          -> (q [R,Hq,512], k [R,Hkv*256], v [R,Hkv*256], idx [R,640])
    choose(out_rows)                 -> list of R token ids (the target's choice after each row)
    mtp_rows(tokens, stacks)         -> (q, k, v, idx) of the draft layer for rows (token p+1, stack of position p)
    draft(mtp_out_row, position)     -> one token id
"""
import torch

from . import capi, layers


class SpecStream:
    """One request: trunk sessions (GDN layers, then one QSA layer), the draft layer's QSA session, token history and
    the ledger of pending rows."""

    def __init__(self, g, gdn_weights, qsa_weights, mtp_weights, glue, ctx, mtp_rows=0, span=9):
        assert 2 <= span <= capi.MAX_STEP_ROWS
        self.g, self.glue, self.span = g, glue, span
        self.gw, self.qw, self.mw = gdn_weights, qsa_weights, mtp_weights
        self.gs = [layers.GdnSession(g, pend_rows=16 if span > 8 else 8) for _ in gdn_weights]
        self.qs = layers.QsaSession(g, ctx, max_rows=capi.MAX_STEP_ROWS)
        self.ms = layers.QsaSession(g, mtp_rows or ctx, max_rows=capi.MAX_STEP_ROWS)     # the draft layer's own cache
        self.mtp_capacity = mtp_rows or ctx
        self.qplan = layers.QsaStepPlan(qsa_weights, capi.MAX_STEP_ROWS)
        self.mplan = layers.QsaStepPlan(mtp_weights, capi.MAX_STEP_ROWS)
        self.tokens = []          # tokens[p] sits at position p; the trunk has processed positions [0, len - 1)
        self.replay = 0           # accepted draft rows that wait in the pending buffers for the next GDN call
        self.mpos = 0             # the draft layer's cache holds rows [0, mpos) made from trunk stacks
        self.stacks = None        # trunk output rows of the positions [mpos, len - 1), for the catch-up rows
        self.accepted = []        # accepted drafts per verify pass

    # ---- trunk -----------------------------------------------------------------------------------------------
    def _trunk(self, tokens, pos0, replay, commit):
        """Rows `tokens` at positions pos0.. through the GDN layers and the QSA layer; returns the QSA output rows."""
        below = None
        for i, (w, s) in enumerate(zip(self.gw, self.gs)):
            qkv, z, x = self.glue.gdn_rows(i, tokens, below)
            below = layers.gdn_step(w, [dict(session=s, qkv=qkv, z=z, x=x, pos0=pos0, replay=replay, commit=commit)])[0]
        q, k, v, idx = self.glue.qsa_rows(tokens, below)
        return self.qplan.run([dict(session=self.qs, q=q, k=k, v=v, idx=idx, pos0=pos0)])[0].clone()

    def feed(self, tokens):
        """Prompt tokens, one trunk row each (all but the last, which opens the first verify span)."""
        for t in tokens:
            if self.tokens:
                out = self._trunk([self.tokens[-1]], len(self.tokens) - 1, self.replay, 1)
                self.replay = 0
                self.stacks = out if self.stacks is None else torch.cat([self.stacks, out])
            self.tokens.append(int(t))

    # ---- draft layer -----------------------------------------------------------------------------------------
    def _mtp(self, tokens, stacks, mpos):
        if not (0 <= mpos and 1 <= len(tokens) <= capi.MAX_STEP_ROWS and mpos + len(tokens) <= self.mtp_capacity):
            raise ValueError("MTP context full or invalid row count")          # ContextRowsFit, engine/runtime/bounds.h:14-16
        q, k, v, idx = self.glue.mtp_rows(tokens, stacks)
        return self.mplan.run([dict(session=self.ms, q=q, k=k, v=v, idx=idx, pos0=mpos)])[0].clone()

    def _draft(self, depth):
        """Catch-up rows for the positions the trunk has finished since the last pass (their stacks are the trunk's own
        outputs), then `depth - 1` chained rows whose stack is the draft layer's previous output."""
        L = len(self.tokens)
        drafts = []
        out = None
        while self.mpos < L - 1:                                   # catch-up in passes of at most 13 rows
            n = min(capi.MAX_STEP_ROWS, L - 1 - self.mpos)
            toks = self.tokens[self.mpos + 1:self.mpos + 1 + n]
            out = self._mtp(toks, self.stacks[:n], self.mpos)
            self.stacks = self.stacks[n:]
            self.mpos += n
        drafts.append(self.glue.draft(out[-1:], L))
        stack = out[-1:]
        for i in range(1, depth):                                  # chained rows: overwritten by the next catch-up
            out = self._mtp([drafts[-1]], stack, self.mpos + i - 1)
            drafts.append(self.glue.draft(out, L + i))
            stack = out
        return drafts

    # ---- one round -------------------------------------------------------------------------------------------
    def round(self, depth=None):
        """Draft, verify, accept.  Returns the tokens the round emitted (accepted drafts + the target's own next token)."""
        depth = depth if depth is not None else self.span - 1
        L = len(self.tokens)
        assert L >= 2 and 1 <= depth <= self.span - 1
        drafts = self._draft(depth)
        rows = [self.tokens[-1]] + drafts
        out = self._trunk(rows, L - 1, self.replay, 1)             # 1 certain row + the drafts, only the first is committed
        preds = self.glue.choose(out)
        n = 0
        while n < depth and drafts[n] == preds[n]:
            n += 1
        self.replay = n                                            # the accepted rows wait in the pending buffers
        self.accepted.append(n)
        emitted = drafts[:n] + [preds[n]]
        self.tokens += emitted
        self.stacks = out[:n + 1] if self.stacks is None or len(self.stacks) == 0 else torch.cat([self.stacks, out[:n + 1]])
        return emitted

    def decode_one(self):
        """Plain decoding: the trunk row of the last token (replaying what is pending), then the target's choice."""
        out = self._trunk([self.tokens[-1]], len(self.tokens) - 1, self.replay, 1)
        self.replay = 0
        self.stacks = out if self.stacks is None or len(self.stacks) == 0 else torch.cat([self.stacks, out])
        self.tokens.append(self.glue.choose(out)[0])
        return self.tokens[-1]

    def flush(self):
        """Applies the pending accepted rows with a one-row trunk pass on the last token, without choosing a token: the
        state then covers every token.  For comparisons at the end of a stream; the stream is not stepped afterwards."""
        out = self._trunk([self.tokens[-1]], len(self.tokens) - 1, self.replay, 1)
        self.replay = 0
        return out
