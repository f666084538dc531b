// crucible_state.hpp — host-side state contracts of the attention path, for an engine that owns its buffers:
// the commit / replay ledger of a sequence, the rules of a speculative verify span, and the one list of a
// sequence's device buffers that every copy (snapshot, restore, checkpoint) walks.  Pure C++17, no CUDA: the
// CPU contract tests compile it with g++ alone.  Names and rules are the reference's
//   RetainedPrefix            engine/runtime/retained_prefix.h:9-50
//   span rules                engine/runtime/spec_span.h:6-64
//   VerifySpan / SpecPrefix   engine/runtime/batch_spec_contract.h:8-40
//   VisitFixedState           engine/model/flashnext/fixed_state.h:11-40
//   QSA cache spans           engine/layers/cache_storage.h:40-46, :75-95; engine/runtime/sequence_state.h:65-82
// with the model geometry as a run-time value (cr_geometry) instead of compile-time constants.
#pragma once
#include <array>
#include <cstddef>
#include <cstdint>
#include <limits>
#include <map>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>
#include "crucible_attn.h"

namespace crucible {

constexpr int kMaxRows = 8;       // rows of one forward / one span of a packed pass (geometry.h:73)
constexpr int kPackedRows = 16;   // rows of one packed multi-session verify pass (geometry.h:74)
constexpr int kSpecSpanMax = CR_MAX_STEP_ROWS;   // 13: the 16-slot rings keep 3 old rows (spec_span.h:6-9)
constexpr int kQsaRawSlots = 16, kQsaRawDim = 128;
static_assert(kSpecSpanMax + 3 <= CR_GDN_HIST_SLOTS, "a span may not overwrite a ring slot the next forward reads");
static_assert(kQsaRawSlots >= kMaxRows + 3, "the raw-key ring keeps the open 4-token block and every verify row");

// ---------------------------------------------------------------------------------------------------------
// Commit / replay ledger.  The recurrent (GDN) state cannot be rolled back: a verify pass stores the state after
// its first `commit` rows and parks the other rows as pending; the next forward must replay exactly the pending
// rows the host kept.  The ledger tracks four counters and refuses every call that would break this.
// ---------------------------------------------------------------------------------------------------------
class RetainedPrefix {
 public:
  // A forward of `rows` new rows that first replays `replay` pending rows and commits its first `commit` rows.
  // Returns "" or the reason the call is refused (the ledger is unchanged then).
  std::string Forward(int rows, int replay, int commit) {
    const bool commit_ok = rows > 0 && commit >= 1 && commit <= rows;
    if (!commit_ok) return "commit must retain at least one row and cannot exceed the forward row count";
    const size_t kept_pending = length_ - committed_;
    const bool replay_ok = replay >= 0 && size_t(replay) == kept_pending && size_t(replay) <= pending_;
    if (!replay_ok) return "replay must equal the retained pending prefix from the previous forward";
    if (std::numeric_limits<size_t>::max() - length_ < size_t(rows)) return "forward length overflow";
    window_start_ = length_;
    committed_ = window_start_ + size_t(commit);
    length_ = window_start_ + size_t(rows);
    pending_ = size_t(rows) - size_t(commit);
    return {};
  }
  // Shrinks the token history to n rows (rejecting drafts).  Committed rows and the first row of the last pass stay.
  std::string Truncate(size_t n) {
    if (n > length_) return "Truncate cannot grow token history";
    if (n == length_) return {};
    if (n == window_start_) return "zero-prefix rollback is unsupported; retain at least one verification row";
    if (n < committed_) return "Truncate cannot cross committed recurrent state";
    length_ = n;
    return {};
  }
  void Reset() { *this = RetainedPrefix(); }
  bool Clean() const { return length_ == 0 && committed_ == 0 && window_start_ == 0 && pending_ == 0; }
  size_t length() const { return length_; }
  size_t committed() const { return committed_; }
  int replay_next() const { return int(length_ - committed_); }   // what the next Forward must pass as `replay`
  // The four counters travel with a snapshot.
  std::array<size_t, 4> Fields() const { return {length_, committed_, window_start_, pending_}; }
  static bool FromFields(const std::array<size_t, 4>& f, RetainedPrefix& out) {
    if (f[1] > f[0] || f[2] > f[0] || f[3] > f[0]) return false;
    out.length_ = f[0]; out.committed_ = f[1]; out.window_start_ = f[2]; out.pending_ = f[3];
    return true;
  }

 private:
  size_t length_ = 0, committed_ = 0, window_start_ = 0, pending_ = 0;
};

// ---------------------------------------------------------------------------------------------------------
// Verify-span rules (all pure).
// ---------------------------------------------------------------------------------------------------------
// Text of the span setting: empty / "8" keeps 8 rows, "9".."13" turn long spans on, anything else is -1.
inline int ResolveSpecSpan(const char* text) {
  if (!text || !*text) return kMaxRows;
  const std::string s(text);
  if (s.size() > 2 || s[0] == '0') return -1;
  int v = 0;
  for (char c : s) {
    if (c < '0' || c > '9') return -1;
    v = v * 10 + (c - '0');
  }
  return v >= kMaxRows && v <= kSpecSpanMax ? v : -1;
}
// Pending GDN rows per head (the stride cr_gdn_step takes as pend_rows).
constexpr int SpecPendRows(int span) { return span > kMaxRows ? kPackedRows : kMaxRows; }
// Draft depth of a request: the API maximum (7) means "as deep as the span allows".
constexpr int SpanDraftDepth(int spec, int span) { return (span > kMaxRows && spec == kMaxRows - 1) ? span - 1 : spec; }
// A lone span may hold `span` rows; the spans of a packed pass keep 8 each.
constexpr bool SpanRowsFit(int rows, int span, int spans) { return rows <= (spans == 1 ? span : kMaxRows); }
// Rows of a span beyond the first 8 are parked in a side buffer by ring users that read 9 old rows.
constexpr bool PleSideRow(int row) { return row >= kMaxRows; }
constexpr int PleSideKeep(int rows, int kept) { return (kept < rows ? kept : rows) > kMaxRows ? (kept < rows ? kept : rows) - kMaxRows : 0; }
// Draft-layer passes (at most 8 rows each, oldest first) that bring `pending` pairs down to `keep` (>= 1).
inline std::vector<int> SpanTrimPasses(int pending, int keep) {
  std::vector<int> passes;
  if (keep < 1) return passes;
  while (pending > keep) {
    const int n = pending - keep < kMaxRows ? pending - keep : kMaxRows;
    passes.push_back(n);
    pending -= n;
  }
  return passes;
}

// One span of a packed verify pass, and the per-stream prefix it extends.
struct VerifySpan {
  int stream;
  std::vector<int> tokens;
  int replay = 0, commit = 1;
};
struct SpecPrefix {
  size_t length;
  int capacity;
  RetainedPrefix retained;
};
// Checks every span of a pass before any stream's ledger changes.  "" = all spans are admissible.
inline std::string SpecSpansError(const std::vector<VerifySpan>& spans, const std::vector<SpecPrefix>& prefixes,
                                  int projection_limit, int temporal_limit, int vocabulary) {
  if (spans.empty() || projection_limit < 1 || temporal_limit < 1 || vocabulary < 1) return "invalid verification limits";
  std::set<int> seen;
  size_t total = 0;
  for (const VerifySpan& s : spans) {
    const bool stream_ok = s.stream >= 0 && size_t(s.stream) < prefixes.size() && seen.insert(s.stream).second;
    if (!stream_ok) return "verification streams must be valid and distinct";
    const size_t n = s.tokens.size();
    if (n == 0 || n > size_t(temporal_limit) || total + n > size_t(projection_limit)) return "verification spans exceed the row limits";
    total += n;
    for (int t : s.tokens)
      if (t < 0 || t >= vocabulary) return "verification token is out of range";
    const SpecPrefix& p = prefixes[size_t(s.stream)];
    if (p.capacity <= 0 || p.length > size_t(p.capacity) || n > size_t(p.capacity) - p.length) return "verification span exceeds its request context";
    RetainedPrefix trial = p.retained;
    const std::string err = trial.Forward(int(n), s.replay, s.commit);
    if (!err.empty()) return err;
  }
  return {};
}

// ---------------------------------------------------------------------------------------------------------
// Byte sizes of the per-sequence buffers for a geometry.
// ---------------------------------------------------------------------------------------------------------
constexpr size_t kGdnScaleFloats = 64;   // per-head lazy scale slots after the state (geometry.h:57)
inline size_t GdnStateBytes(const cr_geometry& g) { return sizeof(float) * (size_t(g.gdn_vheads) * CR_GDN_DIM * CR_GDN_DIM + kGdnScaleFloats); }
inline size_t GdnHistBytes(const cr_geometry& g) {
  return sizeof(float) * CR_GDN_HIST_SLOTS * (2 * size_t(g.gdn_kheads) + size_t(g.gdn_vheads)) * CR_GDN_DIM;
}
inline size_t GdnPendBytes(const cr_geometry& g, int span) { return sizeof(float) * size_t(g.gdn_vheads) * SpecPendRows(span) * CR_PEND_FLOATS; }
// K, V, raw indexer keys, pooled keys of one QSA layer (QsaCacheBytes, cache_storage.h:40-46).
inline std::array<size_t, 4> QsaCacheBytes(const cr_geometry& g, int context, bool bounded) {
  if (context < 1 || context > 1048576) throw std::invalid_argument("QSA cache context is out of range");
  const size_t row = size_t(g.kv_heads) * CR_HEAD_DIM * 2;
  return {size_t(context) * row, size_t(context) * row, size_t(bounded ? kQsaRawSlots : context) * kQsaRawDim * sizeof(float),
          size_t((context + 127) / 128) * 4096 * sizeof(float)};
}

// ---------------------------------------------------------------------------------------------------------
// The one list of a sequence's fixed-size state, in snapshot order: GDN states, raw-row rings, pending rows, then
// `extra` buffers of the host (the reference keeps one more ring there).  State needs maps gstate / ghist / gpend
// from layer to pointer.
// ---------------------------------------------------------------------------------------------------------
struct DeviceSpan { const void* pointer; size_t bytes; };

template <class State, class Add>
void VisitFixedState(const State& state, const cr_geometry& g, size_t pend_bytes, Add&& add) {
  for (const auto& kv : state.gstate) add(kv.second, GdnStateBytes(g));
  for (const auto& kv : state.ghist) add(kv.second, GdnHistBytes(g));
  for (const auto& kv : state.gpend) add(kv.second, pend_bytes);
}
template <class State>
size_t FixedStateBytes(const State& state, const cr_geometry& g, size_t pend_bytes) {
  size_t total = 0;
  VisitFixedState(state, g, pend_bytes, [&](const void*, size_t n) { total += n; });
  return total;
}
template <class State>
bool FixedStateMatches(const State& state, const cr_geometry& g, size_t pend_bytes, size_t expected) {
  return FixedStateBytes(state, g, pend_bytes) == expected;
}

// Per-sequence buffers of the attention path: which layers are QSA (with their caches) and which are GDN.
// The owner allocates; this struct only records pointers and sizes, and lists them.
struct SequenceState {
  cr_geometry geometry{};
  int capacity = 0;                 // positions of every QSA cache
  int span = kMaxRows;              // verify span (8..13): fixes the pending-row stride
  RetainedPrefix retained;
  std::map<int, cr_qsa_cache> qc;   // QSA layers
  std::map<int, float*> gstate, ghist, gpend;   // GDN layers

  size_t PendBytes() const { return GdnPendBytes(geometry, span); }
  size_t FixedBytes() const { return gstate.size() * (GdnStateBytes(geometry) + GdnHistBytes(geometry) + PendBytes()); }
  std::vector<DeviceSpan> FixedSpans() const {
    std::vector<DeviceSpan> v;
    VisitFixedState(*this, geometry, PendBytes(), [&](const void* p, size_t n) { v.push_back({p, n}); });
    return v;
  }
  // Every buffer of the sequence: the four spans of each QSA cache (K, V, raw, pool), then the fixed state.
  std::vector<DeviceSpan> Spans() const {
    std::vector<DeviceSpan> v;
    for (const auto& kv : qc) {
      const cr_qsa_cache& c = kv.second;
      const auto bytes = QsaCacheBytes(geometry, capacity, c.raw_slots != 0);
      v.push_back({c.k, bytes[0]});
      v.push_back({c.v, bytes[1]});
      v.push_back({c.ik_raw, bytes[2]});
      v.push_back({c.ik_pool, bytes[3]});
    }
    for (const DeviceSpan& s : FixedSpans()) v.push_back(s);
    return v;
  }
  // What changes after position p and must be saved for an in-slot checkpoint at p (slot_checkpoint_io.h:14-26):
  // the fixed state, each compact raw ring, and the 128-position pool tile that holds p when p is inside one.
  std::vector<DeviceSpan> CheckpointSpans(size_t position) const {
    std::vector<DeviceSpan> v = FixedSpans();
    for (const auto& kv : qc) {
      const cr_qsa_cache& c = kv.second;
      if (c.raw_slots) v.push_back({c.ik_raw, size_t(c.raw_slots) * kQsaRawDim * sizeof(float)});
      if (position % 128) v.push_back({c.ik_pool + position / 128 * 4096, 4096 * sizeof(float)});
    }
    return v;
  }
  // The spans of a full snapshot that holds `length` positions, in the order a conversation snapshot stores them
  // (engine/runtime/conversation_snapshot.h:47-58): the fixed state first, then per QSA layer K rows, V rows, raw keys
  // (the whole ring when compact) and the pool tiles up to the one that holds length - 1.
  std::vector<DeviceSpan> SnapshotSpans(size_t length) const {
    const size_t row = size_t(geometry.kv_heads) * CR_HEAD_DIM * 2;
    std::vector<DeviceSpan> v = FixedSpans();
    for (const auto& kv : qc) {
      const cr_qsa_cache& c = kv.second;
      if (!length) continue;
      v.push_back({c.k, length * row});
      v.push_back({c.v, length * row});
      v.push_back({c.ik_raw, size_t(c.raw_slots ? c.raw_slots : length) * kQsaRawDim * sizeof(float)});
      v.push_back({c.ik_pool, (length + 127) / 128 * 4096 * sizeof(float)});
    }
    return v;
  }
  // Bytes of a full snapshot that holds `length` positions (QsaSnapshotSpans, cache_storage.h:85-95): K and V rows
  // below length, the raw keys below length (or the whole ring), pool tiles up to the one holding length - 1.
  size_t SnapshotBytes(size_t length) const {
    const size_t row = size_t(geometry.kv_heads) * CR_HEAD_DIM * 2;
    size_t total = FixedBytes();
    for (const auto& kv : qc) {
      const size_t raw = length ? size_t(kv.second.raw_slots ? kv.second.raw_slots : length) * kQsaRawDim * sizeof(float) : 0;
      total += 2 * length * row + raw + (length + 127) / 128 * 4096 * sizeof(float);
    }
    return total;
  }
};

// The same list as the C ABI takes it (cr_state_save / cr_state_restore).
inline std::vector<cr_span> AbiSpans(const std::vector<DeviceSpan>& spans) {
  std::vector<cr_span> v;
  for (const DeviceSpan& s : spans) v.push_back({const_cast<void*>(s.pointer), s.bytes});
  return v;
}

}  // namespace crucible
