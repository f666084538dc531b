// Shared pieces of the chunk-64 WY Gated DeltaNet scan (gdn_chunk_local.cu, gdn_chunk_scan_tc.cu).
//
// The algebra is the reference's chunked form (ref/prefill_ref.py:16-34;
// engine/layers/kernels/prefill_gdn.h:111-249).  Per chunk of 64 tokens and value head, with G the cumulative
// log-decay inside the chunk:
//   L   = tril(beta_i (k_i . k_j) exp(G_i - G_j), -1)        T = (I + L)^-1
//   W   = T (beta e^G K)      Ut = T (beta V)                QKd = tril((q_i . k_j) exp(G_i - G_j))
//   U   = Ut - W S            Y = e^G (Q S) + QKd U          S <- e^{G_end} S + (K e^{G_end - G})^T U
// exp(-G) is never formed.  Products use tf32 operands (rounded to nearest when written) with fp32
// accumulation; the carried state is fp32; the triangular inverse is exact fp32.  tf32 keeps the recurrent
// state within 1e-3 relative of the fp64 oracle (3.4e-4 over 4096 tokens); single-pass bf16 does not (3e-3).
#pragma once
#include "gdn_prefill.cuh"

namespace cr {

constexpr int kChunk = 64;
constexpr int kLdK = 132;   // [64][128] operand read row-major as A, or as B stored [n][k]: stride % 32 == 4
constexpr int kLdX = 136;   // [64][128] operand read as B stored [k][n], or as transposed A: stride % 32 == 8
constexpr int kLdM = 68;    // [64][64] operand read row-major as A

struct ChunkWs {
  float* Ut;   // [Hv][chunks][4][4][128][4] fp32 = [token / 16][(token % 16) / 4][column][token % 4]
  float* G;    // [Hv][chunks][64]         cumulative log decay inside the chunk
  float* WQ;   // [Hv][chunks][32][128][4] rows 0-63 W, rows 64-127 e^G Q, one K-major tf32 tile
  float* QKp;  // [Hv][chunks][16][64][4]  QKd as a K-major tf32 tile
  float* Kt;   // [Hv][chunks][16][128][4] (e^{G_end - G} K)^T as a K-major tf32 tile
  int chunks;
};

__device__ __forceinline__ void mma_tf32(float (&d)[4], const float (&a)[4], float b0, float b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])), "r"(__float_as_uint(a[3])),
        "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// acc[16 x 8NT] += A[16 x 8KT] B.  A row-major in shared memory (lda % 32 == 4), or A_T: stored [k][m]
// (lda % 32 == 8).  B stored [k][n] (ldb % 32 == 8), or B_NK: stored [n][k] (ldb % 32 == 4).
// Operands hold tf32-rounded values.  Bank-conflict free for the stated strides.
template <int NT, int KT, bool A_T, bool B_NK>
__device__ __forceinline__ void warp_gemm(float (&acc)[NT][4], const float* A, int lda, const float* B, int ldb) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int kk = 0; kk < KT; ++kk) {
    float a[4];
    if constexpr (!A_T) {
      a[0] = A[g * lda + kk * 8 + t];       a[1] = A[(g + 8) * lda + kk * 8 + t];
      a[2] = A[g * lda + kk * 8 + t + 4];   a[3] = A[(g + 8) * lda + kk * 8 + t + 4];
    } else {
      a[0] = A[(kk * 8 + t) * lda + g];     a[1] = A[(kk * 8 + t) * lda + g + 8];
      a[2] = A[(kk * 8 + t + 4) * lda + g]; a[3] = A[(kk * 8 + t + 4) * lda + g + 8];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      float b0, b1;
      if constexpr (B_NK) {
        b0 = B[(n * 8 + g) * ldb + kk * 8 + t];
        b1 = B[(n * 8 + g) * ldb + kk * 8 + t + 4];
      } else {
        b0 = B[(kk * 8 + t) * ldb + n * 8 + g];
        b1 = B[(kk * 8 + t + 4) * ldb + n * 8 + g];
      }
      mma_tf32(acc[n], a, b0, b1);
    }
  }
}

// Four 8 x 4 pieces of tf32 values (8 rows of 16 bytes each) in one instruction: lane L passes the address of row
// L % 8 of piece L / 8 and receives element (L / 4, L % 4) of every piece, which is the layout of the m16n8k8
// fragments.  Rows must be 16-byte aligned.
__device__ __forceinline__ void ldmatrix4(float (&v)[4], const float* row) {
  unsigned r0, r1, r2, r3;
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"((unsigned)__cvta_generic_to_shared(row)));
  v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1); v[2] = __uint_as_float(r2); v[3] = __uint_as_float(r3);
}
// Address of this lane's row for the A fragment of rows [0, 16) x k [k0, k0 + 8) of a row-major tile.
__device__ __forceinline__ const float* ldm_a_row(const float* A, int lda, int k0) {
  const int lane = threadIdx.x & 31, j = lane >> 3, r = lane & 7;
  return A + ((j & 1) * 8 + r) * lda + k0 + (j >> 1) * 4;
}

// acc[16 x 8NT] += A B^T with A [16][8KT] and B [8NT][8KT] both row-major over k (strides % 32 == 4), fragments
// by ldmatrix: one instruction for A and one per two column tiles of B per k step.  NT even.
template <int NT, int KT>
__device__ __forceinline__ void warp_gemm_nk_ldm(float (&acc)[NT][4], const float* A, int lda, const float* B, int ldb,
                                                 int n_used = NT) {   // column tiles [n_used, NT) are left untouched (n_used even)
  const int lane = threadIdx.x & 31, j = lane >> 3, r = lane & 7;
  const float* arow = ldm_a_row(A, lda, 0);
  const float* brow = B + ((j >> 1) * 8 + r) * ldb + (j & 1) * 4;
#pragma unroll
  for (int kk = 0; kk < KT; ++kk) {
    float a[4];
    ldmatrix4(a, arow + kk * 8);
#pragma unroll
    for (int n = 0; n < NT; n += 2) {
      if (n >= n_used) break;
      float b[4];
      ldmatrix4(b, brow + n * 8 * ldb + kk * 8);
      mma_tf32(acc[n], a, b[0], b[1]);
      mma_tf32(acc[n + 1], a, b[2], b[3]);
    }
  }
}

// Two products with a lower-triangular A (64 x 64, row-major, lda % 32 == 4) at once: acc_hi = A[rows of block
// m_hi] B and acc_lo = A[rows of block m_lo] B for 8 NT columns of B ([k][n], ldb % 32 == 8), m_lo < m_hi.  Row
// block m only needs k < 16 (m + 1), and the B fragments of the common k range are loaded once.  Pairing blocks
// (3, 0) and (2, 1) gives every warp ten k steps.  ROUND_A: A holds fp32 values that are rounded to tf32 as they are loaded.
template <int NT, bool ROUND_A>
__device__ __forceinline__ void warp_gemm_tril_pair(float (&acc_hi)[NT][4], float (&acc_lo)[NT][4], const float* A, int lda,
                                                    int m_hi, int m_lo, const float* B, int ldb) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const float* Ah = ldm_a_row(A + m_hi * 16 * lda, lda, 0);   // this lane's fragment rows
  const float* Al = ldm_a_row(A + m_lo * 16 * lda, lda, 0);
  const int k_hi = 2 * (m_hi + 1), k_lo = 2 * (m_lo + 1);
#pragma unroll 2
  for (int kk = 0; kk < k_hi; ++kk) {
    const bool both = kk < k_lo;
    float ah[4], al[4] = {0.f, 0.f, 0.f, 0.f};
    ldmatrix4(ah, Ah + kk * 8);
    if (both) ldmatrix4(al, Al + kk * 8);
    if constexpr (ROUND_A) {
#pragma unroll
      for (int i = 0; i < 4; ++i) { ah[i] = tf32r(ah[i]); al[i] = tf32r(al[i]); }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const float b0 = B[(kk * 8 + t) * ldb + n * 8 + g], b1 = B[(kk * 8 + t + 4) * ldb + n * 8 + g];
      mma_tf32(acc_hi[n], ah, b0, b1);
      if (both) mma_tf32(acc_lo[n], al, b0, b1);
    }
  }
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

cr_status gdn_chunk_local_launch(const cr_geometry* g, const GdnPrefillParams& P, const ChunkWs& ws, bool bf16_in, cudaStream_t stream);
cr_status gdn_chunk_scan_tc_launch(const cr_geometry* g, const GdnPrefillParams& P, const ChunkWs& ws, cudaStream_t stream);
size_t gdn_chunk_layout(const cr_geometry* g, int rows, ChunkWs* ws, char* base);

}  // namespace cr
