/* crucible_attn.h — C ABI of the B200 (sm_100a) attention hot path: QSA sparse gated attention and
 * Gated DeltaNet, as a drop-in behind the engine's layer entry points.
 *
 * Conventions
 *  - Every pointer inside an argument struct is a DEVICE pointer owned by the caller (the engine owns
 *    caches, state and scratch: engine/runtime/sequence_state.h:84-112, engine/engine.hip:190-207).
 *    The argument structs themselves live in HOST memory and are copied into kernel parameters.
 *    No entry point allocates device memory.
 *  - Work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the default stream) and the call
 *    returns without synchronising, like the reference launchers.
 *  - Contract violations are reported BEFORE any device write as CR_ERR_INVALID (the reference prints and
 *    aborts: engine/layers/kernels/prefill_qsa.h:250-253, :277-283); cr_last_error() gives the text.
 *  - `spans` arrays batch independent sequences (sessions, or the spans of a packed verify pass) into one
 *    launch chain, the role of PackedStateArgs / PackedQsaArgs (engine/layers/packed_state.h:6-9,
 *    engine/layers/ops.h:448-460).
 *  - fp16 / bf16 buffers are passed as uint16_t* (raw bits).
 */
#ifndef CRUCIBLE_ATTN_H_
#define CRUCIBLE_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  CR_OK = 0,
  CR_ERR_INVALID = 1,      /* argument contract violated; nothing was launched */
  CR_ERR_CUDA = 2,         /* a CUDA runtime call failed */
  CR_ERR_UNSUPPORTED = 3,  /* valid in the reference, not built here (e.g. mrope) */
  CR_ERR_TIMEOUT = 4       /* a bounded device-side wait gave up (status word) */
} cr_status;

/* Model geometry (engine/model/flashnext/geometry.h:47-72).  Fixed by the kernels: head_dim 256, indexer
 * 4 heads x 128, rotary dims 64 (theta 1e7), block 4 tokens, 512 selected blocks, GDN head dim 128,
 * conv width 4.  Variable: the head counts and the hidden width (a/b GEMV length). */
typedef struct {
  int hidden;      /* kHidden: 2560 reference, 2048 benchmark configs */
  int q_heads;     /* kQHeads: 24 / 16 */
  int kv_heads;    /* kKvHeads: 2 */
  int gdn_vheads;  /* kGdnHeads: 48 / 32 */
  int gdn_kheads;  /* kGdnKeyHeads: 16 */
} cr_geometry;

enum { CR_HEAD_DIM = 256, CR_IDX_HEADS = 4, CR_IDX_DIM = 128, CR_ROT_DIM = 64, CR_BLOCK = 4,
       CR_SEL_BLOCKS = 512, CR_GDN_DIM = 128, CR_GDN_CONV = 4, CR_GDN_HIST_SLOTS = 16,
       CR_PEND_FLOATS = 258 /* kPend, engine/layers/ops.h:231 */,
       CR_QSA_SPLITS = 32 /* kQsaSplits, engine/layers/qsa_long.h:389-392 */,
       CR_QSA_PART = 258 /* kQsaPart: m, l, acc[256], engine/layers/qsa_long.h:395 */,
       CR_MAX_STEP_ROWS = 13 /* rows of one decode/verify span: ring headroom, engine/runtime/spec_span.h:6-9 */,
       CR_MAX_PREFILL_ROWS = 2048 /* kPrefillCoreRows, engine/runtime/prefill_rows.h:7 */,
       CR_ROPE_TABLE_FLOATS = 64 /* kRopeTableFloats, engine/layers/ops.h:464 */ };

/* Output format of a layer core. */
typedef enum {
  CR_OUT_RAW_F32 = 0,   /* gated output, fp32 [R][H*D] (for plain-weight out-projections) */
  CR_OUT_RAW_BF16 = 1,  /* gated output, bf16 [R][H*D] */
  CR_OUT_EXL3_WHT = 2   /* the reference's out-projection input: fp16(WHT128(RoundH(RoundH(o)*suh))/sqrt(128)),
                           row-major or the packed GEMM layout (engine/layers/ops.h:224-229, :372-386) */
} cr_out_format;

typedef enum { CR_IN_F32 = 0, CR_IN_BF16 = 1 } cr_in_dtype;

/* ---------------------------------------------------------------------------------------------------
 * Gated DeltaNet
 * ------------------------------------------------------------------------------------------------- */

/* Replaces struct GdnArgs (engine/layers/ops.h:204-222). */
typedef struct {
  const void* qkv;         /* [R][2*Hk*128 + Hv*128] raw projection rows (fp32; bf16 allowed in prefill) */
  const void* z;           /* [R][Hv*128] */
  const float* x;          /* [R][hidden] mixer input, for the a/b projections (decode/verify only) */
  const uint16_t* ab;      /* fp16 [2*Hv][hidden]: rows 0..Hv-1 a, Hv..2Hv-1 b */
  const float* conv;       /* [channels][4] */
  const float* A_log;      /* [Hv] */
  const float* dt_bias;    /* [Hv] */
  const float* gamma;      /* [128] direct gamma */
  float* hist;             /* [16][channels] ring of raw qkv rows, slot = pos & 15 */
  float* state;            /* [Hv][128 key][128 value] fp32, followed by 64 scale floats */
  const uint16_t* suh_out; /* fp16 [Hv*128], CR_OUT_EXL3_WHT only */
  void* out;               /* [R][Hv*128] in the chosen cr_out_format (xh_out in the reference) */
  float* pend;             /* [Hv][pend_rows][258] speculative rows: khat, v, decay, beta */
  int pos0, R;
  int replay;              /* pending rows of the previous forward to fold in first */
  int commit;              /* rows of this forward whose state update is certain (>= 1) */
  int pack_rows, pack_off; /* CR_OUT_EXL3_WHT: >0 selects the packed GEMM layout [c/16][pack_rows][16] */
} cr_gdn_args;

/* Replaces LaunchGdnCore / LaunchGdnSpan / LaunchGdnVerify and the packed verify launch
 * (engine/layers/gdn_rows.h:15-32; engine/layers/gdn_verify.h:428-434;
 * engine/runtime/batch_spec_forward.h:163-176).  One launch serves all spans.
 * pend_rows: pending-row stride per head (8 = kMaxRows, 16 = kPackedRows).
 * Limits: 1 <= R <= CR_MAX_STEP_ROWS, 1 <= commit <= R, 0 <= replay <= pend_rows, R - commit <= pend_rows. */
cr_status cr_gdn_step(const cr_geometry* g, const cr_gdn_args* spans, int n_spans, int pend_rows,
                      cr_out_format fmt, void* stream);

/* Prefill algorithms. */
typedef enum {
  CR_GDN_SERIAL_F32 = 0,  /* exact fp32 token-serial scan (the role of GdnPersistentColumnKernel,
                             engine/layers/kernels/prefill_gdn.h:285-315) */
  CR_GDN_CHUNK_TC = 1     /* chunk-64 WY form, scan on tcgen05 tensor cores with the recurrent operands and the
                             accumulators in tensor memory
                             (LaunchGdnPrefill / LaunchGdnMicro, engine/layers/kernels/prefill_gdn.h:1229-1279).
                             Up to 3 value heads per key head (both model geometries); more: CR_ERR_UNSUPPORTED */
} cr_gdn_algo;

/* Replaces struct GdnPrefill (engine/layers/kernels/prefill_gdn.h:12-29).  input.replay = 0,
 * input.commit = input.R, input.pend unused, input.x / input.ab unused (a/b logits come precomputed). */
typedef struct {
  cr_gdn_args input;
  const void* ab_logits;    /* [R][2*Hv] a then b (fp32 or bf16 per in_dtype) */
  cr_in_dtype in_dtype;     /* dtype of input.qkv, input.z and ab_logits */
  void* workspace;          /* cr_gdn_prefill_workspace_bytes(g, R) bytes */
  size_t workspace_bytes;
  float* raw_y;             /* optional fp32 [R][Hv*128] un-gated readout, for validation; may be NULL */
} cr_gdn_prefill_args;

/* Scratch for one call of `rows` rows: the intermediates of one internal part (7,104 rows, about 72 KB per row),
 * twice that when the call is longer than a part (consecutive parts work on two workspaces in turn). */
size_t cr_gdn_prefill_workspace_bytes(const cr_geometry* g, int rows);
/* 1 when this build of the library carries the algorithm. */
int cr_gdn_algo_available(cr_gdn_algo algo);
/* The internal parts a CR_GDN_CHUNK_TC call of `rows` rows runs in: writes up to max_parts (first row, row count)
 * pairs and returns the number of parts (host only, no device work).  Every part but the last is a multiple of 64
 * rows and none exceeds the part the workspace is sized for.  No counterpart in the reference, whose callers
 * cut the sequence into 2,048-row parts themselves. */
int cr_gdn_prefill_parts(int rows, int* first_row, int* n_rows, int max_parts);

/* Replaces LaunchGdnScanGate / LaunchGdnLanes / LaunchGdnPrefill / LaunchGdnMicro + GdnPrefillHistoryKernel
 * (engine/layers/kernels/prefill_gdn.h:1206-1216, :1161, :1229-1279, :274-282): rows pos0..pos0+R-1 of one
 * layer from the carried state; writes the gated output, the new state and the raw-row ring.
 * Any R >= 1 is accepted (the engine calls it with parts of <= 2048 rows).
 * With CR_GDN_CHUNK_TC a call longer than one internal part runs its kernels on three library-owned streams
 * (created on first use, one set per device) that fork from `stream` and join it again with events before the
 * call returns: to the caller the work is still asynchronous on `stream`, and it can be captured into a graph.
 * Calls on one device are serialised while they enqueue.  With stage timing on everything stays on `stream`. */
cr_status cr_gdn_prefill(const cr_geometry* g, const cr_gdn_prefill_args* a, cr_gdn_algo algo,
                         cr_out_format fmt, void* stream);

/* Replaces LaunchGdnMaterialize (engine/layers/kernels/prefill_gdn.h:48-67): S *= c for heads whose stored
 * lazy scale c is neither 0 nor 1, then c = 1.  `states` is a HOST array of device state pointers. */
cr_status cr_gdn_materialize(const cr_geometry* g, float* const* states, int n_states, void* stream);

/* ---------------------------------------------------------------------------------------------------
 * QSA sparse gated attention
 * ------------------------------------------------------------------------------------------------- */

/* Replaces struct QsaCache (engine/layers/ops.h:407-413). */
typedef struct {
  uint16_t* k;     /* fp16 [ctx][Hkv][256] */
  uint16_t* v;     /* fp16 [ctx][Hkv][256] */
  float* ik_raw;   /* fp32 [ctx][128], or a ring of raw_slots rows */
  float* ik_pool;  /* fp32 tiles [ceil(ctx/128)][128][32]: offset(b,d) = (b/32)*4096 + d*32 + b%32 */
  int raw_slots;   /* 0 keeps the full-prefix layout */
} cr_qsa_cache;

/* Replaces struct QsaArgs (engine/layers/ops.h:422-446). */
typedef struct {
  float* q;               /* [R][Hq][512]: per head [q 256 | gate 256]; q is normed + roped IN PLACE */
  const float* k;         /* [R][Hkv*256] */
  const float* v;         /* [R][Hkv*256] */
  float* idx;             /* [R][640]: 4x128 indexer queries (normed in place) | 128 raw key */
  const float* q_norm1;   /* (1 + w) [256] */
  const float* k_norm1;   /* (1 + w) [256] */
  const float* iq_norm1;  /* (1 + w) [128] */
  const float* ik_norm1;  /* (1 + w) [128] */
  cr_qsa_cache c;
  float* scores;          /* [R][sstride] */
  int sstride;            /* >= (pos0 + R) / 4 */
  int* sel;               /* [R][512] selected block ids, ascending */
  int* nsel;              /* [R]: -1 = dense, else 512 */
  const uint16_t* suh_o;  /* fp16 [Hq*256], CR_OUT_EXL3_WHT only */
  void* out;              /* [R][Hq*256] in the chosen cr_out_format (xh_o in the reference) */
  int pos0, R;
  float* context;         /* optional un-gated fp32 [R][Hq][256] */
  int pack_rows, pack_off;
  const int* mrope;       /* NULL for text; else [capacity][4] (t, h, w, unused) positions of every cache position
                             (SequenceState::mrope, engine/runtime/sequence_state.h:33-35; Rope64Axes, ops.h:515-541) */
  const float* rope;      /* 64-float table: [0,32) inverse frequencies, [32] cos/sin multiplier (plain or YaRN) */
} cr_qsa_args;

/* Scratch sizing (engine/layers/qsa_long.h:226, :396; engine/layers/ops.h:420;
 * engine/layers/cache_storage.h:40-46). */
size_t cr_qsa_scratch_bytes(const cr_geometry* g, int rows);         /* split-KV partials: rows x Hq x 32 x 258 floats
                                                                        (a pass of many rows uses fewer splits of it) */
size_t cr_qsa_select_scratch_bytes(const cr_geometry* g, int rows);  /* 0: the select kernels keep their candidate
                                                                        lists on chip; kept so that
                                                                        QsaSelectScratchFloats call sites compile */
size_t cr_qsa_pool_floats(int ctx);
cr_status cr_qsa_cache_bytes(const cr_geometry* g, int ctx, int bounded, size_t out_bytes[4]);

/* Replaces RopePlainFillKernel / PlainRopeTable (engine/layers/ops.h:469-493). */
cr_status cr_rope_table_fill(float* table, void* stream);
/* The YaRN rows of FillRopeTables (engine/layers/ops.h:476-484; engine/layers/rope_tables.h; RopeMode Yarn2 / Yarn4,
 * engine/runtime/rope_mode.h:13-21): the table for contexts of factor x 262,144 positions, computed instead of stored.
 * factor 1 gives the plain table. */
cr_status cr_rope_table_fill_yarn(float* table, int factor, void* stream);

/* Replaces QsaPrepKernel + QsaPoolKernel (+ QsaRetainRawKernel) for decode / verify rows
 * (engine/layers/ops.h:561-601, :610-645): q and indexer-query heads normed + roped in place, K/V rows to the
 * fp16 cache, raw indexer key cached, blocks completed by these rows pooled. */
cr_status cr_qsa_prep(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void* stream);

/* The query half of cr_qsa_prep alone (q and indexer-query heads normed + roped in place, nothing cached), for up to
 * 2048 rows.  No counterpart in the reference. */
cr_status cr_qsa_prep_queries(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void* stream);

/* Replaces LaunchQsaSelect (engine/layers/qsa_long.h:383-387): indexer scores (rows with more than 512
 * complete blocks) + exact top-512 in the order (score desc, block id asc), emitted ascending;
 * nsel = -1 for dense rows. `scratch` may be NULL when cr_qsa_select_scratch_bytes() is 0. */
cr_status cr_qsa_select(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void* scratch,
                        size_t scratch_bytes, void* stream);

/* Replaces LaunchQsaAttn / QsaAttnTailKernel (engine/layers/qsa_long.h:399-534): split-KV attention over the
 * attended positions, log-sum-exp merge, sigmoid gate, output transform.  `scratch` holds
 * cr_qsa_scratch_bytes(g, total rows) bytes of split-KV partials; it needs no initialisation (every record the
 * merge reads is written by the same call first).  Two launches: the split kernel, then a merge kernel; no
 * block waits on another block and there are no counters (the reference's `sync` words have no counterpart). */
cr_status cr_qsa_attn(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void* scratch,
                      size_t scratch_bytes, cr_out_format fmt, void* stream);

/* No counterpart in the reference (its engine always owns scratch).  Same work and output as cr_qsa_attn, for
 * callers that cannot allocate device memory or pass scratch: a serving process whose HBM is fully committed to
 * caches, a plugin without access to its host's allocator, or a caller that must not allocate while a stream
 * capture is open.  The split-KV partials live in an array inside the library (8.45 MB per GPU, held until the
 * process exits).  Limit: total rows x q_heads <= CR_STATIC_ATTN_MAX_ROW_HEADS, else CR_ERR_INVALID.  All calls on
 * a device share the array: calls whose kernels may overlap on the GPU race.  The first call on a device resolves
 * the array's address; make it before any stream capture starts. */
enum { CR_STATIC_ATTN_MAX_ROW_HEADS = 256 };
cr_status cr_qsa_attn_static(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cr_out_format fmt,
                             void* stream);

/* prep + select + attn, the whole AttentionCore of a QSA layer for decode / verify
 * (engine/runtime/batch_forward.h:300-333). */
cr_status cr_qsa_step(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void* scratch,
                      size_t scratch_bytes, cr_out_format fmt, void* stream);

/* Replaces struct QsaPrefill (engine/layers/kernels/prefill_qsa.h:24-32). */
typedef struct {
  cr_qsa_args input;
  uint16_t* q_hi;         /* fp16 [R][Hq][256] normed + roped queries (written) */
  void* scratch;          /* cr_qsa_prefill_scratch_bytes(g, R) bytes */
  size_t scratch_bytes;
} cr_qsa_prefill_args;

size_t cr_qsa_prefill_scratch_bytes(const cr_geometry* g, int rows);

/* Replaces struct QsaUnion (engine/layers/kernels/prefill_qsa_union.h:18-21).  A tile is cr_qsa_union_tile_rows(g)
 * consecutive rows (128 / query heads per KV head: 16 or 10; the reference uses 4).  list: per tile
 * cr_qsa_union_list_ints(g, rows) / tiles ints = pairs (block id, row mask), ascending block ids; bit r of the mask:
 * row r of the tile attends the block (the reference packs block | mask << 24 into one int, which caps the mask at
 * 4 rows).  count: entries per tile.  cr_qsa_prefill builds the lists in its own scratch; cr_qsa_union_build is the
 * stage alone (QsaUnionBuildKernel, prefill_qsa_union.h:25-68), from a->sel / a->nsel / a->pos0 / a->R. */
typedef struct {
  int* list;
  int* count;
} cr_qsa_union;
size_t cr_qsa_union_list_ints(const cr_geometry* g, int rows);   /* QsaUnionListInts, prefill_qsa_union.h:745 */
int cr_qsa_union_tile_rows(const cr_geometry* g);
cr_status cr_qsa_union_build(const cr_geometry* g, const cr_qsa_args* a, const cr_qsa_union* u, void* stream);

/* Replaces LaunchQsaPrefillCache (engine/layers/kernels/prefill_qsa.h:248-260): cache half of a prefill part. */
cr_status cr_qsa_prefill_cache(const cr_geometry* g, const cr_qsa_args* a, void* stream);

/* Replaces LaunchQsaPrefillUnion / LaunchQsaPrefill (engine/layers/kernels/prefill_qsa_union.h:782-807;
 * prefill_qsa.h:274-299): one part of 1..2048 rows against the growing cache: cache rows, query prep, scores,
 * selection, attention with the fused gate.  skip: leading rows that only get cache work (multiple of 16). */
cr_status cr_qsa_prefill(const cr_geometry* g, const cr_qsa_prefill_args* a, int skip, cr_out_format fmt,
                         void* stream);
/* The attention stage of a part alone (LaunchQsaUnionFlashGate, prefill_qsa_union.h:762-778): union lists + tiled
 * attention + gate for rows [skip, R), from selections already in a->input.sel / nsel, prepared queries in a->q_hi
 * and a cache that holds the part.  The stage a bench drives with injected selections. */
cr_status cr_qsa_prefill_attend(const cr_geometry* g, const cr_qsa_prefill_args* a, int skip, cr_out_format fmt,
                                void* stream);

/* ---------------------------------------------------------------------------------------------------
 * Split-KV across devices (no counterpart in the single-device reference; the partial record is the
 * reference's (m, l, acc[256]) of engine/layers/qsa_long.h:442-445 and the candidate stage is its tile pass,
 * qsa_long.h:228-234).
 * ------------------------------------------------------------------------------------------------- */

/* Local candidates of one rank: for each row the top-512 (score, id) among blocks [b0, b1) owned by the rank.
 * cand_scores/cand_ids: [rows][512]; unused slots hold score -1 and id -1. */
cr_status cr_qsa_shard_candidates(const cr_geometry* g, const cr_qsa_args* a, int b0, int b1,
                                  float* cand_scores, int* cand_ids, void* stream);
/* The same with the scoring in front: scores of blocks [b0, b1) only (the rank reads nothing but its own part of the
 * pool; the cache pointers of a->c and a->scores may be bases biased so that absolute positions and block ids index the
 * rank's own storage, in which case a->sstride only has to cover b1 - b0 blocks), then the candidates.  Scores outside
 * [b0, b1) are left untouched. */
cr_status cr_qsa_shard_select(const cr_geometry* g, const cr_qsa_args* a, int b0, int b1,
                              float* cand_scores, int* cand_ids, void* stream);
/* Global selection from the gathered candidates of all ranks [ranks][rows][512]; writes a->sel / a->nsel. */
cr_status cr_qsa_merge_candidates(const cr_geometry* g, const cr_qsa_args* a, int ranks,
                                  const float* cand_scores, const int* cand_ids, void* stream);
/* Attention over the attended positions inside [p0, p1) only; writes one partial (m, l, acc[256]) per
 * (row, head): partials [rows][Hq][258]. */
cr_status cr_qsa_shard_attn(const cr_geometry* g, const cr_qsa_args* a, int p0, int p1, float* partials,
                            void* scratch, size_t scratch_bytes, void* stream);
/* LSE merge of gathered partials [ranks][rows][Hq][258] + gate + output transform. */
cr_status cr_qsa_merge_partials(const cr_geometry* g, const cr_qsa_args* a, int ranks, const float* partials,
                                cr_out_format fmt, void* stream);

/* ---------------------------------------------------------------------------------------------------
 * Diagnostics
 * ------------------------------------------------------------------------------------------------- */
const char* cr_last_error(void);   /* text of the last error on this thread */
int cr_version(void);
/* Every wait inside a kernel of this library (on an mbarrier that a bulk copy or a tensor-core commit completes) is
 * bounded in time.  A wait that runs out sets a bit of a device status word, after which the kernel issues no more
 * copies or tensor-core work, runs to its end, frees its tensor memory and returns: the context stays usable, the
 * outputs of that launch are undefined.  cr_device_status() synchronises the current device and returns the word
 * (0 = no wait has given up since the library was loaded or the word was cleared): bit 0 = tcgen05 GDN scan,
 * bit 1 = tcgen05 QSA scoring, bit 2 = tcgen05 QSA prefill attention, bit 3 = cr_debug_wait_timeout,
 * bit 4 = cr_proj_gemm.
 * cr_device_check() is the same read as a status code: CR_OK or CR_ERR_TIMEOUT (cr_last_error() names the kernel).
 * cr_device_status_clear() zeroes the word.  All three synchronise: call them outside stream capture, e.g. once per
 * forward pass.  No counterpart in the reference, whose waits spin without bound
 * (engine/layers/qsa_long.h:516-518, engine/layers/kernels/prefill_gdn.h:964-979). */
int cr_device_status(void);
cr_status cr_device_check(void);
cr_status cr_device_status_clear(void);

/* Tuning options of the process, in place of environment switches (the reference reads CRUCIBLE_* switches through
 * one registry, engine/switches.h:44-110; build macros CRUCIBLE_QSA_SPLITS etc.).  cr_get_options() returns the
 * current values, cr_set_options() validates and installs new ones; set them before the first launch that they
 * affect and not concurrently with launches. */
typedef struct {
  int gdn_part_chunks;   /* 64-row chunks per internal part of a long cr_gdn_prefill call: 32..4096 (default 111) */
  int pdl;               /* 1 = programmatic dependent launch along the decode chain (default), 0 = plain launches */
  int qsa_score_simt;    /* 1 = prefill scores with fp32 FMAs instead of tcgen05 (default 0; an A/B and debugging aid) */
  int qsa_union_rows;    /* rows per union tile of the prefill attention: 0 = automatic, 8, 16; -1 = row-wise kernel */
} cr_options;
cr_status cr_get_options(cr_options* out);
cr_status cr_set_options(const cr_options* in);
/* ---- projection GEMMs either side of the core ----------------------------------------------------------------
 * One destination of a projection: columns [col0, col0 + cols) of the product go to ptr[row * ld + (col - col0)],
 * as bf16 or, with f32 != 0, as fp32.  Outputs are listed in column order without gaps; cols is a multiple of 32. */
typedef struct {
  void* ptr;
  int col0, cols, ld, f32;
} cr_proj_out;

/* Y[R][N] = X[R][K] W[N][K]^T, bf16 operands (X row-major, W as [out][in] row-major), fp32 accumulation on tcgen05
 * tensor cores, the columns scattered into up to 6 outputs: the input GEMM group of a prefill layer writing the rows
 * the core reads (GDN: qkv | z | a,b logits as bf16 for cr_gdn_prefill with CR_IN_BF16; QSA: q | k | v | idx as fp32)
 * or the output GEMM writing hidden rows (PrefillLayer::input / ::output, engine/runtime/prefill_engine.inc:261-270,
 * :362, for plain bf16 weights; the reference's EXL3 weight decoding is not part of this path, and its GEMM-epilogue
 * form of the GDN q/k prep, engine/layers/kernels/prefill_gdn.h:431-492, lives in the chunk kernel of cr_gdn_prefill
 * here).  K a multiple of 64, N >= 32.  Nothing is allocated; bit 4 of the device status word reports a bounded
 * wait that gave up. */
cr_status cr_proj_gemm(const void* x, const void* w, int R, int K, int N, const cr_proj_out* outs, int n_outs,
                       void* stream);

/* ---- state snapshot / restore --------------------------------------------------------------------------------------
 * A span of device memory in a snapshot list.  The lists themselves (which buffers, in which order) are the host's:
 * include/crucible_state.hpp builds them the way SequenceState::FixedSpans, SlotCheckpointIO::Spans and
 * QsaSnapshotSpans do (engine/runtime/sequence_state.h:56-60; engine/runtime/slot_checkpoint_io.h:14-26;
 * engine/layers/cache_storage.h:85-95). */
typedef struct {
  void* ptr;                     /* 16-byte aligned */
  size_t bytes;                  /* multiple of 16 (every buffer of this path is) */
} cr_span;

/* Sum of the spans' bytes = the size of the buffer a snapshot of them needs (SlotCheckpointIO::Bytes). */
size_t cr_spans_bytes(const cr_span* spans, int n);

/* Copies the spans, in order and back to back, into `buffer` (save) or out of it (restore): the copy loops of
 * SlotCheckpointIO::Save / Restore (engine/runtime/slot_checkpoint_io.h:49-73) and CopySnapshotSpans
 * (engine/runtime/snapshot_bytes.h:692-704) as one kernel per 96 spans on `stream`, in order with the forwards
 * around it.  `buffer` is device memory, or pinned host memory the device can address (a conversation snapshot).
 * The ledger (RetainedPrefix) and the token history that belong to a checkpoint are host data and stay with the
 * caller.  CR_ERR_INVALID if the buffer is smaller than the spans, or a span is not 16-byte aligned and sized. */
cr_status cr_state_save(const cr_span* spans, int n, void* buffer, size_t buffer_bytes, void* stream);
cr_status cr_state_restore(const cr_span* spans, int n, const void* buffer, size_t buffer_bytes, void* stream);

/* Number of kernels this library has launched in this process (for launch accounting in benches). */
unsigned long long cr_kernel_launches(void);

/* Stage timing, the role of Engine::Mark / Engine::Collect under CRUCIBLE_PROFILE (engine/engine.hip:2086-2106):
 * while enabled, one CUDA event is recorded after every kernel the library launches on the calling thread;
 * cr_profile_begin() plants the starting event on `stream`; cr_profile_collect() synchronises on the last
 * event and returns the number of distinct kernels, with names[i*32..], summed milliseconds and launch counts. */
cr_status cr_profile_enable(int on);
cr_status cr_profile_begin(void* stream);
int cr_profile_collect(char* names, float* ms, int* calls, int max_stages);

/* Self-check of the tensor-core (tcgen05) building blocks, exported as a test hook: D[128][N] = A B^T in tf32 on
 * one CTA, A [128][K] and B [N][K] both K-major.  *status (device int) becomes 1 if the bounded wait on the MMA
 * gave up.  No counterpart in the reference. */
cr_status cr_debug_umma_gemm(const float* A, const float* B, float* D, int K, int N, int* status, void* stream);
/* The same self-check for fp16 operands (kind::f16) with the B operand MN-major, i.e. B [K][N] as a V tile lies in the
 * cache (keys x channels, channels contiguous): D[128][N] = A[128][K] B.  variant selects which of the two descriptor
 * strides is the step along N (0) or along K (1); the production kernel uses the one this check confirms. */
cr_status cr_debug_umma_f16_gemm(const uint16_t* A, const uint16_t* B, float* D, int K, int N, int variant, int* status,
                                 void* stream);
/* The same self-check for one step of the tiled prefill attention without its softmax: the K and V rows of 16
 * four-token blocks (ids in `blocks`, device ints) of KV head `head` are copied from fp16 caches [rows][kv_heads][256]
 * by tensor-map (TMA) boxes into 128-byte-swizzled shared-memory tiles; S[128][64] = Q K^T (Q[128][256] from tensor
 * memory, the K tile K-major) and O[128][256] = Pm V (Pm[128][64], the V tile MN-major).  Blocks past `rows` read as
 * zeros.  *status: 1 = a bounded wait gave up, 2 = shared memory not aligned for the swizzle. */
cr_status cr_debug_umma_kv_step(const uint16_t* k_cache, const uint16_t* v_cache, int kv_heads, int rows, int head,
                                const int* blocks, const uint16_t* Q, const uint16_t* Pm, float* S, float* O,
                                int* status, void* stream);
/* Test hook for the bounded waits: one CTA waits up to max_us microseconds on an mbarrier that nothing will ever
 * complete (no copy, no tensor-core work pending), then sets *status (device int) to 1, raises bit 3 of the device
 * status word and returns normally.  Shows that a wait that runs out ends the kernel and leaves the context
 * usable.  max_us in 1..100000.  No counterpart in the reference. */
cr_status cr_debug_wait_timeout(int* status, unsigned max_us, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CRUCIBLE_ATTN_H_ */
