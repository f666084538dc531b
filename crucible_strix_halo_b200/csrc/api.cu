// Error plumbing, geometry validation and diagnostics of the C ABI.
#include <atomic>
#include <cstring>
#include <vector>
#include "common.cuh"

namespace cr {

static thread_local char g_error[512] = "";
static std::atomic<unsigned long long> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

cr_status cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return CR_ERR_CUDA;
}

// ---- stage timing: one event after every kernel launch while profiling is on (the role of Engine::Mark /
// Collect, engine/engine.hip:2086-2106).  Elapsed time of a launch = its event minus the previous event on the
// same thread; cr_profile_begin() plants the first one.
struct Mark { cudaEvent_t ev; const char* name; };
static thread_local std::vector<Mark> g_marks;
static thread_local std::vector<cudaEvent_t> g_pool;
static thread_local cudaStream_t g_stream = nullptr;
static std::atomic<int> g_profile{0};

static void mark(const char* name);
// Called at the top of every launcher: while profiling it also plants a starting event, so the time charged to the
// launcher's first kernel does not include host-side gaps before it.
void use_stream(cudaStream_t stream) {
  g_stream = stream;
  if (g_profile.load(std::memory_order_relaxed)) mark(nullptr);
}

static void mark(const char* name) {
  cudaEvent_t ev;
  if (!g_pool.empty()) { ev = g_pool.back(); g_pool.pop_back(); }
  else if (cudaEventCreate(&ev) != cudaSuccess) return;
  cudaEventRecord(ev, g_stream);
  g_marks.push_back({ev, name});
}

bool profiling() { return g_profile.load(std::memory_order_relaxed) != 0; }

void count_launch(const char* name) {
  g_launches.fetch_add(1ull, std::memory_order_relaxed);
  if (g_profile.load(std::memory_order_relaxed)) mark(name);
}

static cr_options g_options = {kGdnPartChunksDefault, 1, 0, 0};
const cr_options& options() { return g_options; }

cr_status check_geometry(const cr_geometry* g) {
  CR_REQUIRE(g, "null geometry");
  CR_REQUIRE(g->hidden >= 8 && g->hidden % 8 == 0 && g->hidden <= 16384, "geometry: hidden=%d must be a multiple of 8 in 8..16384", g->hidden);
  CR_REQUIRE(g->kv_heads >= 1 && g->kv_heads <= 8, "geometry: kv_heads=%d out of range", g->kv_heads);
  CR_REQUIRE(g->q_heads >= g->kv_heads && g->q_heads % g->kv_heads == 0 && g->q_heads / g->kv_heads >= 8 && g->q_heads / g->kv_heads <= 12,
             "geometry: q_heads=%d must be a multiple of kv_heads=%d with 8..12 query heads per KV head", g->q_heads, g->kv_heads);
  CR_REQUIRE(g->gdn_kheads >= 1 && g->gdn_vheads >= g->gdn_kheads && g->gdn_vheads % g->gdn_kheads == 0 && g->gdn_vheads % 2 == 0 &&
             g->gdn_vheads <= 64, "geometry: gdn heads %d/%d unsupported", g->gdn_vheads, g->gdn_kheads);
  return CR_OK;
}

}  // namespace cr

extern "C" const char* cr_last_error(void) { return cr::g_error; }
extern "C" int cr_version(void) { return 1; }
extern "C" unsigned long long cr_kernel_launches(void) { return cr::g_launches.load(std::memory_order_relaxed); }

extern "C" cr_status cr_get_options(cr_options* out) {
  CR_REQUIRE(out, "cr_get_options: null argument");
  *out = cr::g_options;
  return CR_OK;
}

extern "C" cr_status cr_set_options(const cr_options* in) {
  CR_REQUIRE(in, "cr_set_options: null argument");
  CR_REQUIRE(in->gdn_part_chunks >= 32 && in->gdn_part_chunks <= 4096, "cr_set_options: gdn_part_chunks=%d outside 32..4096", in->gdn_part_chunks);
  CR_REQUIRE(in->pdl == 0 || in->pdl == 1, "cr_set_options: pdl must be 0 or 1");
  CR_REQUIRE(in->qsa_score_simt == 0 || in->qsa_score_simt == 1, "cr_set_options: qsa_score_simt must be 0 or 1");
  CR_REQUIRE(in->qsa_union_rows == 0 || in->qsa_union_rows == 8 || in->qsa_union_rows == 16 || in->qsa_union_rows == -1,
             "cr_set_options: qsa_union_rows must be 0 (automatic), 8, 16 or -1 (row-wise kernel)");
  cr::g_options = *in;
  return CR_OK;
}

extern "C" int cr_device_status(void) {
  return cr::gdn_scan_status_read() | (cr::qsa_score_status_read() << 1) | (cr::qsa_flash_status_read() << 2) |
         (cr::debug_wait_status_read() << 3) | (cr::proj_gemm_status_read() << 4);
}

extern "C" cr_status cr_device_check(void) {
  const int st = cr_device_status();
  if (st == 0) return CR_OK;
  cr::set_error("a bounded device-side wait gave up (status word 0x%x:%s%s%s%s%s); the outputs of that launch are undefined",
                st, st & 1 ? " gdn_chunk_scan_tc_kernel" : "", st & 2 ? " qsa_score_tc_kernel" : "", st & 4 ? " qsa_flash_tc_kernel" : "",
                st & 8 ? " debug_wait_kernel" : "", st & 16 ? " proj_gemm_kernel" : "");
  return CR_ERR_TIMEOUT;
}

extern "C" cr_status cr_device_status_clear(void) {
  cr::gdn_scan_status_clear();
  cr::qsa_score_status_clear();
  cr::qsa_flash_status_clear();
  cr::debug_wait_status_clear();
  cr::proj_gemm_status_clear();
  CR_CUDA(cudaGetLastError());
  return CR_OK;
}

extern "C" cr_status cr_profile_enable(int on) { cr::g_profile.store(on ? 1 : 0); return CR_OK; }

extern "C" cr_status cr_profile_begin(void* stream) {
  cr::use_stream((cudaStream_t)stream);
  if (cr::g_profile.load()) cr::mark(nullptr);
  return CR_OK;
}

extern "C" int cr_profile_collect(char* names, float* ms, int* calls, int max_stages) {
  using namespace cr;
  int n = 0;
  if (!g_marks.empty()) cudaEventSynchronize(g_marks.back().ev);
  for (size_t i = 0; i < g_marks.size(); ++i) {
    const Mark& m = g_marks[i];
    if (m.name && i > 0) {
      float t = 0.f;
      if (cudaEventElapsedTime(&t, g_marks[i - 1].ev, m.ev) == cudaSuccess) {
        int k = 0;
        while (k < n && strncmp(names + 32 * k, m.name, 31) != 0) ++k;
        if (k == n && n < max_stages) { strncpy(names + 32 * k, m.name, 31); names[32 * k + 31] = 0; ms[k] = 0.f; calls[k] = 0; ++n; }
        if (k < n) { ms[k] += t; calls[k] += 1; }
      }
    }
  }
  for (const Mark& m : g_marks) g_pool.push_back(m.ev);
  g_marks.clear();
  return n;
}
