// QSA prefill part (1..2048 rows against the growing cache) for sm_100a: cache rows, query prep, scores,
// selection, attention with the fused gate.  Entry point of a part, in the role of LaunchQsaPrefillUnion /
// LaunchQsaPrefill (engine/layers/kernels/prefill_qsa_union.h:782-807; prefill_qsa.h:274-299).
// Attention runs over row tiles on tcgen05 tensor cores (qsa_flash.cu: union lists + masked flash attention); the
// row-wise split-KV kernel of the decode path (qsa_attn.cu, 4 splits per row) remains as the alternative that
// cr_options.qsa_union_rows = -1 selects.  Rows of a part are independent once the cache and the pool hold the
// part, so causality inside the part falls out of pos0 + r.
#include <climits>
#include "qsa.cuh"

namespace cr {
constexpr int kPrefillSplits = 4;

int qsa_union_rows(const cr_geometry* g);
int qsa_union_cap(int RT);
cr_status qsa_union_build_launch(const cr_geometry* g, const cr_qsa_args& a, int2* list, int* count, cudaStream_t stream);
cr_status qsa_flash_launch(const cr_geometry* g, const cr_qsa_args& a, const __half* q_hi, const int2* list, const int* count,
                           float* gated, cr_out_format fmt, int flash_max, cudaStream_t stream);

// Scratch of a part: [split-KV partials of the row-wise kernels][gated fp32 rows for the EXL3 transform of the tiled
// kernel][union lists, 2 ints per entry][union counts].  The list area is sized for tiles of 8 rows, the smallest tile.
static size_t partial_bytes(const cr_geometry* g, int rows) { return (size_t)rows * g->q_heads * kPrefillSplits * CR_QSA_PART * sizeof(float); }
static size_t gated_bytes(const cr_geometry* g, int rows) { return (size_t)rows * g->q_heads * 256 * sizeof(float); }
static size_t list_ints(int rows) { return (size_t)((rows + 7) / 8) * qsa_union_cap(8) * 2; }
// A tile goes to the tiled tensor-core kernel when its rows share enough blocks: at most this many union entries per
// row of the tile (of 513 possible).  Measured on B200 at 262,144 context: a step of 16 entries costs the tiled kernel
// about 3 us per (tile, KV head) when its gathers miss L2, the row-wise kernels about 69 SM-us per (row, KV head).
constexpr int kFlashEntriesPerRow = 320;

static cr_status check_part(const cr_geometry* g, const cr_qsa_prefill_args* args, int skip, cr_out_format fmt, const char* who) {
  CR_REQUIRE(args, "%s: null args", who);
  if (cr_status s = qsa_validate(g, &args->input, 1, CR_MAX_PREFILL_ROWS, who)) return s;
  const cr_qsa_args& q = args->input;
  CR_REQUIRE(skip >= 0 && skip < q.R && skip % 16 == 0, "%s: skip=%d must be a multiple of 16 below R=%d", who, skip, q.R);
  CR_REQUIRE(fmt == CR_OUT_RAW_F32 || fmt == CR_OUT_RAW_BF16 || fmt == CR_OUT_EXL3_WHT, "%s: bad output format", who);
  CR_REQUIRE(q.out && (fmt != CR_OUT_EXL3_WHT || q.suh_o), "%s: output buffer (and suh_o for the EXL3 output) needed", who);
  CR_REQUIRE(fmt == CR_OUT_EXL3_WHT || q.pack_rows == 0, "%s: packed layout only with the EXL3 output", who);
  const size_t need = cr_qsa_prefill_scratch_bytes(g, q.R - skip);
  CR_REQUIRE(args->scratch && args->scratch_bytes >= need, "%s: scratch of %zu bytes needed, %zu given", who, need, args->scratch_bytes);
  CR_REQUIRE(((uintptr_t)args->scratch & 15) == 0, "%s: scratch must be 16-byte aligned", who);
  return CR_OK;
}

// The rows [skip, R) of a part as an argument block of their own.
static cr_qsa_args output_rows(const cr_geometry* g, cr_qsa_args q, int skip, cr_out_format fmt) {
  const size_t W = (size_t)g->q_heads * 256;
  q.pos0 += skip; q.R -= skip;
  q.q += (size_t)skip * g->q_heads * 512; q.idx += (size_t)skip * 640;
  if (q.context) q.context += (size_t)skip * W;
  if (q.pack_rows) q.pack_off += skip;
  else q.out = (char*)q.out + (size_t)skip * W * (fmt == CR_OUT_RAW_F32 ? 4 : 2);
  return q;
}

// Attention of the output rows with sel / nsel in place.
static cr_status attend(const cr_geometry* g, const cr_qsa_prefill_args* args, const cr_qsa_args& q, int skip, cr_out_format fmt,
                        cudaStream_t stream) {
  char* scratch = (char*)args->scratch;
  if (options().qsa_union_rows >= 0 && args->q_hi) {
    float* gated = reinterpret_cast<float*>(scratch + partial_bytes(g, q.R));
    int2* list = reinterpret_cast<int2*>(scratch + partial_bytes(g, q.R) + gated_bytes(g, q.R));
    int* count = reinterpret_cast<int*>(list + list_ints(q.R) / 2);
    const int RT = qsa_union_rows(g);
    const QsaTileSplit tiles = {count, RT, options().qsa_union_rows > 0 ? INT_MAX : kFlashEntriesPerRow * RT};   // an explicit tile size forces the tiled kernel
    if (cr_status s = qsa_union_build_launch(g, q, list, count, stream)) return s;
    if (cr_status s = qsa_flash_launch(g, q, reinterpret_cast<const __half*>(args->q_hi) + (size_t)skip * g->q_heads * 256, list, count,
                                       gated, fmt, tiles.max, stream)) return s;
    if (tiles.max == INT_MAX) return CR_OK;
    // the tiles with little sharing: row-wise split-KV attention (its CTAs of tiled rows exit at once)
    if (cr_status s = qsa_attn_launch(g, &q, 1, (float*)scratch, kPrefillSplits, 0, INT_MAX, stream, &tiles)) return s;
    return qsa_merge_launch(g, &q, 1, (const float*)scratch, kPrefillSplits, false, nullptr, fmt, stream, &tiles);
  }
  if (cr_status s = qsa_attn_launch(g, &q, 1, (float*)scratch, kPrefillSplits, 0, INT_MAX, stream)) return s;
  return qsa_merge_launch(g, &q, 1, (const float*)scratch, kPrefillSplits, false, nullptr, fmt, stream);
}
}  // namespace cr

extern "C" size_t cr_qsa_prefill_scratch_bytes(const cr_geometry* g, int rows) {
  if (!g || rows < 1) return 0;
  return cr::partial_bytes(g, rows) + cr::gated_bytes(g, rows) + cr::list_ints(rows) * sizeof(int) + (size_t)((rows + 7) / 8) * sizeof(int);
}

extern "C" size_t cr_qsa_union_list_ints(const cr_geometry* g, int rows) {
  if (!g || rows < 1 || cr::check_geometry(g) != CR_OK) return 0;
  const int RT = cr::qsa_union_rows(g);
  return (size_t)((rows + RT - 1) / RT) * cr::qsa_union_cap(RT) * 2;
}

extern "C" int cr_qsa_union_tile_rows(const cr_geometry* g) {
  return g && cr::check_geometry(g) == CR_OK ? cr::qsa_union_rows(g) : 0;
}

extern "C" cr_status cr_qsa_union_build(const cr_geometry* g, const cr_qsa_args* a, const cr_qsa_union* u, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_union_build")) return s;
  CR_REQUIRE(u && u->list && u->count, "cr_qsa_union_build: null list or count");
  CR_REQUIRE(((uintptr_t)u->list & 7) == 0, "cr_qsa_union_build: list must be 8-byte aligned");
  return qsa_union_build_launch(g, *a, reinterpret_cast<int2*>(u->list), u->count, (cudaStream_t)stream);
}

extern "C" cr_status cr_qsa_prefill_attend(const cr_geometry* g, const cr_qsa_prefill_args* args, int skip, cr_out_format fmt, void* stream) {
  using namespace cr;
  if (cr_status s = check_part(g, args, skip, fmt, "cr_qsa_prefill_attend")) return s;
  return attend(g, args, output_rows(g, args->input, skip, fmt), skip, fmt, (cudaStream_t)stream);
}

extern "C" cr_status cr_qsa_prefill(const cr_geometry* g, const cr_qsa_prefill_args* args, int skip, cr_out_format fmt, void* stream_) {
  using namespace cr;
  if (cr_status s = check_part(g, args, skip, fmt, "cr_qsa_prefill")) return s;
  cudaStream_t stream = (cudaStream_t)stream_;
  // cache rows + query prep for the whole part (rows below skip get cache work only)
  if (cr_status s = qsa_prep_launch(g, &args->input, 1, 0, reinterpret_cast<__half*>(args->q_hi), skip, stream)) return s;
  const cr_qsa_args q = output_rows(g, args->input, skip, fmt);
  if (cr_status s = qsa_select_launch(g, &q, 1, stream)) return s;
  return attend(g, args, q, skip, fmt, stream);
}
