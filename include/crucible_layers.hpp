// crucible_layers.hpp — the engine-facing C++ names of the attention core, implemented on the C ABI of
// crucible_attn.h.  A maintainer of the engine includes this header in place of layers/ops.h (GDN/QSA parts),
// layers/qsa_long.h, layers/gdn_rows.h, layers/kernels/prefill_gdn.h and layers/kernels/prefill_qsa*.h; the
// struct fields and launcher names below are the reference's, so call sites keep their shape.
// Differences: launchers take the geometry, return cr_status instead of aborting, and take scratch sizes.
#pragma once
#include <cstddef>
#include <stdexcept>
#include <string>
#include <vector>
#include "crucible_attn.h"

namespace crucible {

using Geometry = cr_geometry;
using GdnArgs = cr_gdn_args;          // engine/layers/ops.h:204-222
using QsaCache = cr_qsa_cache;        // engine/layers/ops.h:407-413
using QsaArgs = cr_qsa_args;          // engine/layers/ops.h:422-446
using GdnPrefill = cr_gdn_prefill_args;  // engine/layers/kernels/prefill_gdn.h:12-29
using QsaPrefill = cr_qsa_prefill_args;  // engine/layers/kernels/prefill_qsa.h:24-32
using QsaUnion = cr_qsa_union;           // engine/layers/kernels/prefill_qsa_union.h:18-21 (list entries are (block, row mask) pairs here)

constexpr int kPend = CR_PEND_FLOATS;            // engine/layers/ops.h:231
constexpr int kSelBlocks = CR_SEL_BLOCKS;        // geometry.h:66
constexpr int kQsaSplits = CR_QSA_SPLITS;        // engine/layers/qsa_long.h:392
constexpr int kQsaPart = CR_QSA_PART;            // engine/layers/qsa_long.h:395
constexpr int kRopeTableFloats = CR_ROPE_TABLE_FLOATS;

// The reference aborts on a contract violation; a host that wants the same behaviour wraps calls in Check().
inline void Check(cr_status s) {
  if (s != CR_OK) throw std::runtime_error(std::string("crucible_attn: ") + cr_last_error());
}

// engine/layers/ops.h:416-420, engine/layers/cache_storage.h:16-18
constexpr size_t QsaPoolOffset(int b, int d) { return (size_t)(b / 32) * 4096 + (size_t)d * 32 + b % 32; }
inline size_t QsaPoolFloats(int ctx) { return cr_qsa_pool_floats(ctx); }
constexpr size_t QsaRawOffset(int slots, int position, int dimension) {
  return (size_t)(slots ? position % slots : position) * 128 + dimension;
}
// engine/layers/qsa_long.h:396, :226
inline size_t QsaScratchBytes(const Geometry& g, int rows) { return cr_qsa_scratch_bytes(&g, rows); }
inline size_t QsaSelectScratchBytes(const Geometry& g, int rows) { return cr_qsa_select_scratch_bytes(&g, rows); }
// engine/layers/ops.h:226-229
constexpr size_t OutProjIndex(int r, int c, int width, int pack_rows, int pack_off) {
  return pack_rows ? ((size_t)(c >> 4) * pack_rows + pack_off + r) * 16 + (c & 15) : (size_t)r * width + c;
}

// engine/layers/ops.h:476-493; the YaRN tables of engine/layers/rope_tables.h by their factor (1 = plain, 2, 4)
inline cr_status FillRopeTables(float* tables, void* stream = nullptr) { return cr_rope_table_fill(tables, stream); }
inline cr_status FillRopeTablesYarn(float* tables, int factor, void* stream = nullptr) { return cr_rope_table_fill_yarn(tables, factor, stream); }

// ---- Gated DeltaNet ----------------------------------------------------------------------------------
// engine/layers/gdn_rows.h:26-32 (state_cache is a gfx1151 cache-policy hint and is ignored here).
inline cr_status LaunchGdnCore(const Geometry& g, const GdnArgs& a, int /*state_cache*/ = 0, void* stream = nullptr,
                               int pend_rows = 8, cr_out_format fmt = CR_OUT_EXL3_WHT) {
  return cr_gdn_step(&g, &a, 1, pend_rows, fmt, stream);
}
// Packed verify: one launch for every span of a pass (engine/runtime/batch_spec_forward.h:163-176).
inline cr_status LaunchGdnSpans(const Geometry& g, const GdnArgs* spans, int n, void* stream = nullptr, int pend_rows = 16,
                                cr_out_format fmt = CR_OUT_EXL3_WHT) {
  return cr_gdn_step(&g, spans, n, pend_rows, fmt, stream);
}
// engine/layers/kernels/prefill_gdn.h:1206-1216 (default scan) and :1229-1279 (chunk-64 WY)
inline cr_status LaunchGdnScanGate(const Geometry& g, const GdnPrefill& a, void* stream = nullptr,
                                   cr_out_format fmt = CR_OUT_EXL3_WHT) {
  return cr_gdn_prefill(&g, &a, cr_gdn_algo_available(CR_GDN_CHUNK_TC) ? CR_GDN_CHUNK_TC : CR_GDN_SERIAL_F32, fmt, stream);
}
inline cr_status LaunchGdnPrefill(const Geometry& g, const GdnPrefill& a, void* stream = nullptr,
                                  cr_out_format fmt = CR_OUT_EXL3_WHT) {
  return cr_gdn_prefill(&g, &a, CR_GDN_CHUNK_TC, fmt, stream);
}
// engine/layers/kernels/prefill_gdn.h:60-67
inline cr_status LaunchGdnMaterialize(const Geometry& g, const std::vector<float*>& states, void* stream = nullptr) {
  return cr_gdn_materialize(&g, states.data(), (int)states.size(), stream);
}

// ---- QSA ---------------------------------------------------------------------------------------------
// QsaPrepKernel + QsaPoolKernel + LaunchQsaRetainRaw (engine/runtime/batch_forward.h:309-318)
inline cr_status LaunchQsaPrep(const Geometry& g, const QsaArgs* spans, int n, void* stream = nullptr) {
  return cr_qsa_prep(&g, spans, n, stream);
}
// engine/layers/qsa_long.h:383-387
inline cr_status LaunchQsaSelect(const Geometry& g, const QsaArgs& a, void* scratch = nullptr, size_t scratch_bytes = 0,
                                 void* stream = nullptr) {
  return cr_qsa_select(&g, &a, 1, scratch, scratch_bytes, stream);
}
// engine/layers/qsa_long.h:531-534 and QsaAttnTailKernel (:508-528)
inline cr_status LaunchQsaAttn(const Geometry& g, const QsaArgs& a, void* scratch, size_t scratch_bytes, void* stream = nullptr,
                               cr_out_format fmt = CR_OUT_EXL3_WHT) {
  return cr_qsa_attn(&g, &a, 1, scratch, scratch_bytes, fmt, stream);
}
// The whole AttentionCore of a QSA layer for every span of a pass (PackedQsaCore, batch_spec_forward.h:226-253).
inline cr_status LaunchQsaStep(const Geometry& g, const QsaArgs* spans, int n, void* scratch, size_t scratch_bytes,
                               void* stream = nullptr, cr_out_format fmt = CR_OUT_EXL3_WHT) {
  return cr_qsa_step(&g, spans, n, scratch, scratch_bytes, fmt, stream);
}
// engine/layers/kernels/prefill_qsa.h:248-260
inline cr_status LaunchQsaPrefillCache(const Geometry& g, const QsaArgs& q, void* stream = nullptr) {
  return cr_qsa_prefill_cache(&g, &q, stream);
}
// engine/layers/kernels/prefill_qsa_union.h:782-807; mark(name) is replaced by cr_profile_enable/collect.
inline cr_status LaunchQsaPrefillUnion(const Geometry& g, const QsaPrefill& a, void* stream = nullptr, int skip = 0,
                                       cr_out_format fmt = CR_OUT_EXL3_WHT) {
  return cr_qsa_prefill(&g, &a, skip, fmt, stream);
}

// engine/layers/kernels/prefill_qsa_union.h:745-748 (ints of the list area for `rows` output rows) and :25-68
inline size_t QsaUnionListInts(const Geometry& g, int rows) { return cr_qsa_union_list_ints(&g, rows); }
inline cr_status LaunchQsaUnionBuild(const Geometry& g, const QsaArgs& a, const QsaUnion& u, void* stream = nullptr) {
  return cr_qsa_union_build(&g, &a, &u, stream);
}
// Attention of a part whose cache rows, queries and selections are in place (the QsaUnionStageKernel launch of
// LaunchQsaPrefillUnion, prefill_qsa_union.h:795-806).
inline cr_status LaunchQsaPrefillAttend(const Geometry& g, const QsaPrefill& a, void* stream = nullptr, int skip = 0,
                                        cr_out_format fmt = CR_OUT_EXL3_WHT) {
  return cr_qsa_prefill_attend(&g, &a, skip, fmt, stream);
}

}  // namespace crucible
