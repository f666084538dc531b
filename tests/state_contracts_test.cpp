// CPU contract cases of include/crucible_state.hpp, following the reference's own host tests
// (tests/retained_prefix_test.cpp, tests/spec_span_test.cpp, tests/fixed_state_test.cpp, tests/cache_storage_test.cpp):
// commit / replay / truncate rules of the ledger, the verify-span rules, the visit order and byte totals of the
// fixed state, the QSA cache sizes.  Built and run by tests/test_state_contracts.py with g++ (no CUDA).
#include "../include/crucible_state.hpp"
#include <cassert>
#include <cstdio>
#include <string>
#include <vector>

using namespace crucible;

static bool has(const std::string& s, const char* what) { return s.find(what) != std::string::npos; }

static void ledger_cases() {
  RetainedPrefix s;
  assert(s.Clean());
  assert(has(s.Forward(8, 0, 0), "at least one"));       // a pass must commit a row
  assert(has(s.Forward(8, 0, 9), "commit"));              // more commits than rows
  assert(has(s.Forward(8, 1, 8), "replay"));              // nothing is pending yet
  assert(s.Clean());                                       // refused calls change nothing
  assert(s.Forward(8, 0, 8).empty());
  assert(has(s.Truncate(0), "zero-prefix"));
  assert(has(s.Truncate(7), "committed"));
  assert(has(s.Truncate(9), "grow"));
  assert(s.Forward(8, 0, 1).empty());                      // a verify pass: 1 certain row + 7 drafts
  assert(has(s.Truncate(8), "zero-prefix"));
  assert(s.Truncate(12).empty());                          // 3 drafts accepted
  assert(s.replay_next() == 3);
  assert(has(s.Forward(1, 2, 1), "replay"));
  assert(has(s.Forward(1, 4, 1), "replay"));
  assert(s.Forward(1, 3, 1).empty());
  assert(has(s.Truncate(12), "zero-prefix"));
  // every depth and acceptance of a single-session verification loop
  for (int depth = 1; depth < 8; ++depth)
    for (int accepted = 0; accepted <= depth; ++accepted) {
      RetainedPrefix c;
      assert(c.Forward(8, 0, 8).empty());
      assert(c.Forward(8, 0, 8).empty());
      assert(c.Forward(depth + 1, 0, 1).empty());
      assert(c.Truncate(16 + accepted + 1).empty());
      assert(c.replay_next() == accepted);
      assert(c.Forward(3, accepted, 1).empty());
      assert(c.Truncate(16 + accepted + 2).empty());
      assert(c.Forward(1, 0, 1).empty());
    }
  // 13-row spans (pending stride 16): 12 drafts, any acceptance
  for (int accepted = 0; accepted <= 12; ++accepted) {
    RetainedPrefix c;
    assert(c.Forward(100, 0, 100).empty());
    assert(c.Forward(13, 0, 1).empty());
    assert(c.Truncate(100 + 1 + accepted).empty());
    assert(has(c.Forward(13, accepted + 1, 1), "replay"));
    assert(c.Forward(13, accepted, 1).empty());
  }
  // the counters travel with a snapshot
  RetainedPrefix t;
  assert(RetainedPrefix::FromFields(s.Fields(), t) && t.Fields() == s.Fields());
  assert(!RetainedPrefix::FromFields({4, 5, 0, 0}, t) && !RetainedPrefix::FromFields({4, 0, 5, 0}, t) &&
         !RetainedPrefix::FromFields({4, 0, 0, 5}, t));
  s.Reset();
  assert(s.Clean() && s.Forward(1, 0, 1).empty());
}

static void span_cases() {
  static_assert(kMaxRows == 8 && kSpecSpanMax == 13 && kSpecSpanMax <= kPackedRows, "span limits");
  assert(ResolveSpecSpan(nullptr) == 8 && ResolveSpecSpan("") == 8 && ResolveSpecSpan("8") == 8);
  for (int n = 9; n <= 13; ++n) assert(ResolveSpecSpan(std::to_string(n).c_str()) == n);
  for (const char* bad : {"0", "1", "7", "14", "16", "17", "-9", "+9", " 9", "9 ", "09", "9x", "on", "1.0"})
    assert(ResolveSpecSpan(bad) == -1);
  assert(SpecPendRows(8) == 8);
  for (int n = 9; n <= kSpecSpanMax; ++n) assert(SpecPendRows(n) == 16 && SpecPendRows(n) >= n - 1);
  for (int spec = 0; spec <= 7; ++spec) assert(SpanDraftDepth(spec, 8) == spec);
  assert(SpanDraftDepth(7, 13) == 12 && SpanDraftDepth(7, 9) == 8 && SpanDraftDepth(6, 13) == 6 && SpanDraftDepth(0, 13) == 0);
  assert(SpanRowsFit(1, 13, 1) && SpanRowsFit(13, 13, 1) && !SpanRowsFit(14, 13, 1));
  assert(SpanRowsFit(8, 13, 2) && !SpanRowsFit(9, 13, 2) && !SpanRowsFit(9, 8, 1));
  assert(!PleSideRow(0) && !PleSideRow(7) && PleSideRow(8) && PleSideRow(12));
  assert(PleSideKeep(13, 1) == 0 && PleSideKeep(13, 8) == 0 && PleSideKeep(13, 9) == 1 && PleSideKeep(13, 13) == 5 &&
         PleSideKeep(9, 9) == 1 && PleSideKeep(8, 8) == 0);
  assert(SpanTrimPasses(8, 8).empty() && SpanTrimPasses(1, 8).empty() && SpanTrimPasses(13, 13).empty());
  assert(SpanTrimPasses(9, 1) == std::vector<int>{8} && SpanTrimPasses(13, 8) == std::vector<int>{5});
  assert(SpanTrimPasses(14, 6) == std::vector<int>{8} && (SpanTrimPasses(17, 1) == std::vector<int>{8, 8}));
  assert(SpanTrimPasses(3, 0).empty());

  // a packed pass is validated as a whole before any ledger moves (batch_spec_contract.h)
  std::vector<SpecPrefix> px(3);
  for (auto& p : px) { p.length = 100; p.capacity = 4096; assert(p.retained.Forward(100, 0, 100).empty()); }
  std::vector<VerifySpan> ok = {{0, {1, 2, 3}, 0, 1}, {2, {4, 5, 6, 7, 8, 9, 10, 11}, 0, 1}};
  assert(SpecSpansError(ok, px, 16, 8, 1000).empty());
  assert(has(SpecSpansError({}, px, 16, 8, 1000), "limits"));
  assert(has(SpecSpansError({{0, {1}, 0, 1}, {0, {2}, 0, 1}}, px, 16, 8, 1000), "distinct"));
  assert(has(SpecSpansError({{3, {1}, 0, 1}}, px, 16, 8, 1000), "distinct"));
  assert(has(SpecSpansError({{0, std::vector<int>(9, 1), 0, 1}}, px, 16, 8, 1000), "row limits"));
  assert(has(SpecSpansError({{0, std::vector<int>(8, 1), 0, 1}, {1, std::vector<int>(8, 1), 0, 1}, {2, {1}, 0, 1}}, px, 16, 8, 1000), "row limits"));
  assert(has(SpecSpansError({{0, {1000}, 0, 1}}, px, 16, 8, 1000), "out of range"));
  assert(has(SpecSpansError({{0, {1}, 2, 1}}, px, 16, 8, 1000), "replay"));
  assert(has(SpecSpansError({{0, {1}, 0, 0}}, px, 16, 8, 1000), "at least one"));
  px[1].length = 4090;
  assert(has(SpecSpansError({{1, std::vector<int>(8, 1), 0, 1}}, px, 16, 8, 1000), "context"));
}

static void layout_cases() {
  const cr_geometry ref = {2560, 24, 2, 48, 16}, bench = {2048, 16, 2, 32, 16};
  // reference geometry: 3 MiB of state + 64 scale floats, a 16-row ring of 10,240 channels
  assert(GdnStateBytes(ref) == sizeof(float) * (48 * 128 * 128 + 64));
  assert(GdnHistBytes(ref) == sizeof(float) * 16 * 10240);
  assert(GdnStateBytes(bench) == sizeof(float) * (32 * 128 * 128 + 64) && GdnHistBytes(bench) == sizeof(float) * 16 * 8192);
  assert(GdnPendBytes(ref, 8) == sizeof(float) * 48 * 8 * 258 && GdnPendBytes(ref, 13) == sizeof(float) * 48 * 16 * 258);
  const auto full = QsaCacheBytes(ref, 262144, false), ring = QsaCacheBytes(ref, 262144, true);
  assert(full[0] == 262144u * 1024 && full[1] == full[0] && full[2] == 262144u * 512 && full[3] == 2048u * 4096 * 4);
  assert(ring[2] == 16u * 512 && ring[3] == full[3]);
  assert(QsaCacheBytes(ref, 1, false)[3] == 4096u * 4 && QsaCacheBytes(ref, 129, false)[3] == 2u * 4096 * 4);
  bool threw = false;
  try { QsaCacheBytes(ref, 0, false); } catch (const std::invalid_argument&) { threw = true; }
  assert(threw);

  // the visit order is the snapshot layout: states, rings, pending rows; the total follows the formula, and a
  // buffer missing from one map fails the match
  static float cells[3 * 36];
  SequenceState st;
  st.geometry = ref;
  st.capacity = 4096;
  for (int layer = 0; layer < 36; ++layer) {
    st.gstate[layer] = cells + layer;
    st.ghist[layer] = cells + 36 + layer;
    st.gpend[layer] = cells + 72 + layer;
  }
  std::vector<const void*> order;
  VisitFixedState(st, ref, st.PendBytes(), [&](const void* p, size_t) { order.push_back(p); });
  assert(order.size() == 108 && order.front() == cells && order[36] == cells + 36 && order[72] == cells + 72 && order.back() == cells + 107);
  const size_t total = 36 * (GdnStateBytes(ref) + GdnHistBytes(ref) + st.PendBytes());
  assert(st.FixedBytes() == total && FixedStateBytes(st, ref, st.PendBytes()) == total && FixedStateMatches(st, ref, st.PendBytes(), total));
  st.gpend.erase(35);
  assert(!FixedStateMatches(st, ref, st.PendBytes(), total));
  st.gpend[35] = cells + 107;

  // QSA caches come first in the full list, four spans each; checkpoints add the ring and the open pool tile
  static float kv[4];
  cr_qsa_cache c = {reinterpret_cast<uint16_t*>(kv), reinterpret_cast<uint16_t*>(kv + 1), kv + 2, kv + 3, 0};
  st.qc[3] = c;
  c.raw_slots = 16;
  st.qc[7] = c;
  const auto spans = st.Spans();
  assert(spans.size() == 8 + 108 && spans[0].bytes == 4096u * 1024 && spans[2].bytes == 4096u * 512 && spans[6].bytes == 16u * 512);
  assert(spans[3].bytes == 32u * 4096 * 4 && spans[8].pointer == cells);
  assert(st.CheckpointSpans(256).size() == 108 + 1);                    // on a tile boundary: only the compact ring
  const auto cp = st.CheckpointSpans(300);
  assert(cp.size() == 108 + 3 && cp.back().pointer == kv + 3 + 2 * 4096 && cp.back().bytes == 4096u * 4);
  assert(st.SnapshotBytes(0) == total);
  assert(st.SnapshotBytes(130) == total + 2 * (2 * 130u * 1024 + 2u * 4096 * 4) + 130u * 512 + 16u * 512);
  // the span list of a full snapshot adds up to the same bytes, fixed state first, and converts to the ABI's spans
  const auto snap = st.SnapshotSpans(130);
  size_t sum = 0;
  for (const auto& s : snap) sum += s.bytes;
  assert(snap.size() == 108 + 8 && snap.front().pointer == cells && sum == st.SnapshotBytes(130));
  assert(snap[108].bytes == 130u * 1024 && snap[110].bytes == 130u * 512 && snap[114].bytes == 16u * 512 && snap[115].bytes == 2u * 4096 * 4);
  assert(st.SnapshotSpans(0).size() == 108);
  const auto abi = AbiSpans(snap);
  assert(abi.size() == snap.size() && abi[110].ptr == kv + 2 && abi[110].bytes == snap[110].bytes);
}

int main() {
  ledger_cases();
  span_cases();
  layout_cases();
  std::puts("state_contracts_test: ok");
  return 0;
}
