// Chunk-64 WY Gated DeltaNet scan for sm_100a on tensor cores (tf32 operands, fp32 accumulation and state).
//
// The algebra is the reference's chunked form (ref/prefill_ref.py:16-34;
// engine/layers/kernels/prefill_gdn.h:111-249).  Per chunk of 64 tokens and value head, with G the cumulative
// log-decay inside the chunk:
//   L   = tril(beta_i (k_i . k_j) exp(G_i - G_j), -1)        T = (I + L)^-1
//   W   = T (beta e^G K)      Ut = T (beta V)                QKd = tril((q_i . k_j) exp(G_i - G_j))
//   U   = Ut - W S            Y = e^G (Q S) + QKd U          S <- e^{G_end} S + (K e^{G_end - G})^T U
// exp(-G) is never formed.
//
// Two kernels:
//   gdn_chunk_local_kernel  everything that does not depend on the carried state (Gram matrices, the
//       triangular inverse, W, Ut, QKd), fully parallel over (chunk, key head); the value heads of a key head
//       share its Gram matrices.  Products run as mma.sync m16n8k8 tf32; the 64x64 unit-triangular inverse is
//       exact fp32 forward substitution, one thread per column, no barriers.
//   gdn_chunk_scan_kernel   the sequential part: one CTA per (value head, 32-column slice of the state), state
//       slice in accumulator registers (fp32) for the whole call, operands of the next chunk streamed with
//       cp.async while the current chunk is multiplied.  Warps 0-3 run the recurrence chain (W S, U, K^T U),
//       warps 4-7 the readout (Q S, QKd U), so the readout is off the critical path.
// tf32 (10-bit mantissa, round-to-nearest on every operand write) keeps the recurrent state within 1e-3
// relative of the fp64 oracle; single-pass bf16 does not (3e-3 on 4096 tokens).
#include "gdn_prefill.cuh"

namespace cr {

constexpr int kChunk = 64;

__device__ __forceinline__ void mma_tf32(float (&d)[4], const float (&a)[4], float b0, float b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])), "r"(__float_as_uint(a[3])),
        "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// acc[16 x 8NT] += A[16 x 8KT] B.  A row-major in shared memory (lda % 32 == 4), or A_T: stored [k][m]
// (lda % 32 == 8).  B stored [k][n] (ldb % 32 == 8), or B_NK: stored [n][k] (ldb % 32 == 4).
// All operands already hold tf32-rounded values.  Bank-conflict free for the stated strides.
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

struct ChunkWs {
  float* W;    // [Hv][chunks][64][128]
  float* Ut;   // [Hv][chunks][64][128]
  float* QKd;  // [Hv][chunks][64][64]
  float* G;    // [Hv][chunks][64]
  int chunks;
};

// ------------------------------------------------------------------------------------------------------
// local (state-independent) part: grid (chunks, Hk), 256 threads
// ------------------------------------------------------------------------------------------------------
constexpr int kLdK = 132, kLdX = 136, kLdM = 68;
constexpr size_t kLocalSmem = (size_t)(64 * kLdK + 64 * kLdX + 4 * 64 * kLdM + 3 * 64 + 16 * 64) * sizeof(float);

__global__ void __launch_bounds__(256) gdn_chunk_local_kernel(GdnPrefillParams P, ChunkWs ws) {
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm;                       // [64][132] khat (tf32)
  float* Qx = Ks + 64 * kLdK;           // [64][132] qhat, later [64][136] X = beta e^G K / beta V
  float* KKs = Qx + 64 * kLdX;          // [64][68] K K^T (fp32)
  float* QKs = KKs + 64 * kLdM;         // [64][68] Q K^T (fp32)
  float* Ls = QKs + 64 * kLdM;          // [64][68] strictly lower L
  float* Ts = Ls + 64 * kLdM;           // [64][68] T = (I + L)^-1 (tf32)
  float* Gs = Ts + 64 * kLdM;           // [64] cumulative log decay
  float* bs = Gs + 64;                  // [64] beta
  float* es = bs + 64;                  // [64] beta * exp(G)
  float* Ms = es + 64;                  // [16][64] scratch of the blocked inverse
  const int c = blockIdx.x, kh = blockIdx.y;
  const int t = threadIdx.x, w = t >> 5, l = t & 31, g = l >> 2, tq = l & 3;
  const int R = P.a.R, r0 = c * kChunk, valid = min(kChunk, R - r0);
  const int rep = P.Hv / P.Hk, VW = P.Hv * 128;

  for (int i = t; i < 64 * 32; i += 256) {
    const int row = i >> 5, c4 = (i & 31) * 4;
    float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), qv = kv;
    if (row < valid) {
      kv = *reinterpret_cast<const float4*>(P.kn + ((size_t)(r0 + row) * P.Hk + kh) * 128 + c4);
      qv = *reinterpret_cast<const float4*>(P.qn + ((size_t)(r0 + row) * P.Hk + kh) * 128 + c4);
    }
    *reinterpret_cast<float4*>(Ks + row * kLdK + c4) = make_float4(tf32r(kv.x), tf32r(kv.y), tf32r(kv.z), tf32r(kv.w));
    *reinterpret_cast<float4*>(Qx + row * kLdK + c4) = make_float4(tf32r(qv.x), tf32r(qv.y), tf32r(qv.z), tf32r(qv.w));
  }
  __syncthreads();
  {   // Gram matrices: warps 0-3 K K^T, warps 4-7 Q K^T; 16 rows each
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    const int mt = w & 3;
    warp_gemm<8, 16, false, true>(acc, (w < 4 ? Ks : Qx) + mt * 16 * kLdK, kLdK, Ks, kLdK);
    float* dst = (w < 4 ? KKs : QKs) + (mt * 16) * kLdM;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      *reinterpret_cast<float2*>(dst + g * kLdM + n * 8 + 2 * tq) = make_float2(acc[n][0], acc[n][1]);
      *reinterpret_cast<float2*>(dst + (g + 8) * kLdM + n * 8 + 2 * tq) = make_float2(acc[n][2], acc[n][3]);
    }
  }
  __syncthreads();

  for (int vi = 0; vi < rep; ++vi) {
    const int h = kh * rep + vi;
    const size_t unit = (size_t)h * ws.chunks + c;
    if (w == 0) {   // cumulative log decay of the chunk (padding rows: g = 0, beta = 0)
      const int i0 = 2 * l, i1 = 2 * l + 1;
      const float g0 = i0 < valid ? P.glog[(size_t)(r0 + i0) * P.Hv + h] : 0.f;
      const float g1 = i1 < valid ? P.glog[(size_t)(r0 + i1) * P.Hv + h] : 0.f;
      float s = g0 + g1;
#pragma unroll
      for (int step = 1; step < 32; step <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, s, step);
        if (l >= step) s += v;
      }
      const float G1 = s, G0 = s - g1;
      const float b0 = i0 < valid ? P.beta[(size_t)(r0 + i0) * P.Hv + h] : 0.f;
      const float b1 = i1 < valid ? P.beta[(size_t)(r0 + i1) * P.Hv + h] : 0.f;
      Gs[i0] = G0; Gs[i1] = G1; bs[i0] = b0; bs[i1] = b1;
      es[i0] = b0 * __expf(G0); es[i1] = b1 * __expf(G1);
      ws.G[unit * 64 + i0] = G0; ws.G[unit * 64 + i1] = G1;
    }
    __syncthreads();
    float* qkd = ws.QKd + unit * 64 * 64;
    for (int i = t; i < 64 * 64; i += 256) {
      const int row = i >> 6, col = i & 63;
      const float pair = col <= row ? __expf(Gs[row] - Gs[col]) : 0.f;
      Ls[row * kLdM + col] = col < row ? bs[row] * KKs[row * kLdM + col] * pair : 0.f;
      qkd[i] = tf32r(QKs[row * kLdM + col] * pair);
    }
    for (int i = t; i < 64 * 32; i += 256) {   // X = beta e^G K
      const int row = i >> 5, c4 = (i & 31) * 4;
      const float4 kv = *reinterpret_cast<const float4*>(Ks + row * kLdK + c4);
      const float e = es[row];
      *reinterpret_cast<float4*>(Qx + row * kLdX + c4) = make_float4(tf32r(e * kv.x), tf32r(e * kv.y), tf32r(e * kv.z), tf32r(e * kv.w));
    }
    __syncthreads();
    // T = (I + L)^-1 in exact fp32, blocked 16x16.  Diagonal blocks by forward substitution (one thread per
    // column, column in registers); block row a below the diagonal is T_a = -T_aa (L_a T_above).
    for (int i = t; i < 64 * 64; i += 256) Ts[(i >> 6) * kLdM + (i & 63)] = 0.f;
    __syncthreads();
    if (t < 64) {
      const int b = t >> 4, j = t & 15;
      float D[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = (i == j) ? 1.f : 0.f;
#pragma unroll
        for (int m = 0; m < i; ++m) acc = fmaf(-Ls[(16 * b + i) * kLdM + 16 * b + m], D[m], acc);
        D[i] = acc;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) Ts[(16 * b + i) * kLdM + 16 * b + j] = D[i];
    }
    __syncthreads();
    for (int a = 1; a < 4; ++a) {
      const int wid = 16 * a;                    // columns left of the diagonal block
      for (int e = t; e < 16 * wid; e += 256) {  // M = L_a T_above
        const int i = e / wid, j = e % wid;
        float acc = 0.f;
        for (int m = j & ~15; m < wid; ++m) acc = fmaf(Ls[(wid + i) * kLdM + m], Ts[m * kLdM + j], acc);
        Ms[i * 64 + j] = acc;
      }
      __syncthreads();
      for (int e = t; e < 16 * wid; e += 256) {  // T_a = -T_aa M
        const int i = e / wid, j = e % wid;
        float acc = 0.f;
        for (int m = 0; m <= i; ++m) acc = fmaf(Ts[(wid + i) * kLdM + wid + m], Ms[m * 64 + j], acc);
        Ts[(wid + i) * kLdM + j] = -acc;
      }
      __syncthreads();
    }
    for (int i = t; i < 64 * 64; i += 256) {
      float* p = Ts + (i >> 6) * kLdM + (i & 63);
      *p = tf32r(*p);
    }
    __syncthreads();
    const int mt = w & 3, nh = w >> 2;
    {   // W = T X
      float acc[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      warp_gemm<8, 8, false, false>(acc, Ts + mt * 16 * kLdM, kLdM, Qx + nh * 64, kLdX);
      float* dst = ws.W + (unit * 64 + mt * 16) * 128 + nh * 64;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        *reinterpret_cast<float2*>(dst + g * 128 + n * 8 + 2 * tq) = make_float2(tf32r(acc[n][0]), tf32r(acc[n][1]));
        *reinterpret_cast<float2*>(dst + (g + 8) * 128 + n * 8 + 2 * tq) = make_float2(tf32r(acc[n][2]), tf32r(acc[n][3]));
      }
    }
    __syncthreads();
    for (int i = t; i < 64 * 32; i += 256) {   // X = beta V
      const int row = i >> 5, c4 = (i & 31) * 4;
      float4 vv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < valid) vv = *reinterpret_cast<const float4*>(P.vn + (size_t)(r0 + row) * VW + h * 128 + c4);
      const float b = bs[row];
      *reinterpret_cast<float4*>(Qx + row * kLdX + c4) = make_float4(tf32r(b * vv.x), tf32r(b * vv.y), tf32r(b * vv.z), tf32r(b * vv.w));
    }
    __syncthreads();
    {   // Ut = T X  (kept in fp32: it is added, not multiplied, in the scan)
      float acc[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      warp_gemm<8, 8, false, false>(acc, Ts + mt * 16 * kLdM, kLdM, Qx + nh * 64, kLdX);
      float* dst = ws.Ut + (unit * 64 + mt * 16) * 128 + nh * 64;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        *reinterpret_cast<float2*>(dst + g * 128 + n * 8 + 2 * tq) = make_float2(acc[n][0], acc[n][1]);
        *reinterpret_cast<float2*>(dst + (g + 8) * 128 + n * 8 + 2 * tq) = make_float2(acc[n][2], acc[n][3]);
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------------
// scan: grid Hv*4, 256 threads
// ------------------------------------------------------------------------------------------------------
constexpr int kLdS = 40;   // 32-column slices, stride % 32 == 8
constexpr size_t kScanSmem =
    (size_t)(2 * 64 * kLdK /* W, Q */ + 64 * kLdS /* Ut */ + 64 /* G */ + 64 * kLdX /* K */ + 64 * kLdM /* QKd */ +
             128 * kLdS /* S operand */ + 2 * 64 * kLdS /* U, U' */) * sizeof(float);

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

__global__ void __launch_bounds__(256) gdn_chunk_scan_kernel(GdnPrefillParams P, ChunkWs ws) {
  extern __shared__ __align__(16) float sm[];
  float* Wsm = sm;                       // [64][132]
  float* Qsm = Wsm + 64 * kLdK;          // [64][132]
  float* Utsm = Qsm + 64 * kLdK;         // [64][40]
  float* Gsm = Utsm + 64 * kLdS;         // [64]
  float* Ksm = Gsm + 64;                 // [64][136]  khat, read transposed
  float* QKsm = Ksm + 64 * kLdX;         // [64][68]
  float* Sop = QKsm + 64 * kLdM;         // [128][40]  tf32 copy of the state slice
  float* Usm = Sop + 128 * kLdS;         // [64][40]
  float* Upsm = Usm + 64 * kLdS;         // [64][40]   e^{G_end - G} U
  const int t = threadIdx.x, w = t >> 5, l = t & 31, g = l >> 2, tq = l & 3;
  const int h = blockIdx.x >> 2, col0 = (blockIdx.x & 3) * 32;
  const int rep = P.Hv / P.Hk, kh = h / rep, VW = P.Hv * 128, R = P.a.R;
  const int nch = ws.chunks;

  auto load_a = [&](int c) {   // W, Q, Ut slice, G of chunk c
    const size_t unit = (size_t)h * nch + c;
    const int r0 = c * kChunk;
    const float* Wg = ws.W + unit * 64 * 128;
    for (int i = t; i < 64 * 32; i += 256) {
      const int row = i >> 5, c4 = (i & 31) * 4;
      cp_async16(Wsm + row * kLdK + c4, Wg + row * 128 + c4, true);
      const bool ok = r0 + row < R;
      cp_async16(Qsm + row * kLdK + c4, P.qn + ((size_t)(ok ? r0 + row : 0) * P.Hk + kh) * 128 + c4, ok);
    }
    const float* Ug = ws.Ut + unit * 64 * 128 + col0;
    for (int i = t; i < 64 * 8; i += 256) {
      const int row = i >> 3, c4 = (i & 7) * 4;
      cp_async16(Utsm + row * kLdS + c4, Ug + row * 128 + c4, true);
    }
    if (t < 16) cp_async16(Gsm + t * 4, ws.G + unit * 64 + t * 4, true);
  };
  auto load_b = [&](int c) {   // K, QKd of chunk c
    const size_t unit = (size_t)h * nch + c;
    const int r0 = c * kChunk;
    for (int i = t; i < 64 * 32; i += 256) {
      const int row = i >> 5, c4 = (i & 31) * 4;
      const bool ok = r0 + row < R;
      cp_async16(Ksm + row * kLdX + c4, P.kn + ((size_t)(ok ? r0 + row : 0) * P.Hk + kh) * 128 + c4, ok);
    }
    const float* Qg = ws.QKd + unit * 64 * 64;
    for (int i = t; i < 64 * 16; i += 256) {
      const int row = i >> 4, c4 = (i & 15) * 4;
      cp_async16(QKsm + row * kLdM + c4, Qg + row * 64 + c4, true);
    }
  };

  // state slice: warp w < 4 owns key rows [32w, 32w+32) x 32 columns as two 16-row accumulator tiles
  float S[2][4][4];
  float* st = P.a.state + (size_t)h * 16384 + col0;
  if (w < 4) {
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int row = 32 * w + 16 * mi + g, col = 8 * n + 2 * tq;
        const float2 lo = *reinterpret_cast<const float2*>(st + (size_t)row * 128 + col);
        const float2 hi = *reinterpret_cast<const float2*>(st + (size_t)(row + 8) * 128 + col);
        S[mi][n][0] = lo.x; S[mi][n][1] = lo.y; S[mi][n][2] = hi.x; S[mi][n][3] = hi.y;
        *reinterpret_cast<float2*>(Sop + row * kLdS + col) = make_float2(tf32r(lo.x), tf32r(lo.y));
        *reinterpret_cast<float2*>(Sop + (row + 8) * kLdS + col) = make_float2(tf32r(hi.x), tf32r(hi.y));
      }
  }
  load_a(0);
  cp_async_commit();

  for (int c = 0; c < nch; ++c) {
    cp_async_wait_all();
    __syncthreads();                       // group A of chunk c and the state operand are visible
    load_b(c);
    cp_async_commit();
    const int mt = w & 3;
    const float Gend = Gsm[63];
    const float Glo = Gsm[mt * 16 + g], Ghi = Gsm[mt * 16 + g + 8];
    float acc[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    // Q is rounded here (the prep workspace holds fp32): the tf32 unit ignores the low mantissa bits
    warp_gemm<4, 16, false, false>(acc, (w < 4 ? Wsm : Qsm) + mt * 16 * kLdK, kLdK, Sop, kLdS);
    if (w < 4) {   // U = Ut - W S; keep U (tf32) and U' = e^{G_end - G} U for the state update
      const float slo = __expf(Gend - Glo), shi = __expf(Gend - Ghi);
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = 8 * n + 2 * tq;
        const float2 ulo = *reinterpret_cast<const float2*>(Utsm + (mt * 16 + g) * kLdS + col);
        const float2 uhi = *reinterpret_cast<const float2*>(Utsm + (mt * 16 + g + 8) * kLdS + col);
        const float u0 = ulo.x - acc[n][0], u1 = ulo.y - acc[n][1], u2 = uhi.x - acc[n][2], u3 = uhi.y - acc[n][3];
        *reinterpret_cast<float2*>(Usm + (mt * 16 + g) * kLdS + col) = make_float2(tf32r(u0), tf32r(u1));
        *reinterpret_cast<float2*>(Usm + (mt * 16 + g + 8) * kLdS + col) = make_float2(tf32r(u2), tf32r(u3));
        *reinterpret_cast<float2*>(Upsm + (mt * 16 + g) * kLdS + col) = make_float2(tf32r(slo * u0), tf32r(slo * u1));
        *reinterpret_cast<float2*>(Upsm + (mt * 16 + g + 8) * kLdS + col) = make_float2(tf32r(shi * u2), tf32r(shi * u3));
      }
    } else {       // readout part 1: e^G (Q S)
      const float elo = __expf(Glo), ehi = __expf(Ghi);
#pragma unroll
      for (int n = 0; n < 4; ++n) { acc[n][0] *= elo; acc[n][1] *= elo; acc[n][2] *= ehi; acc[n][3] *= ehi; }
    }
    cp_async_wait_all();
    __syncthreads();                       // U, U' and group B visible; W / Q / Ut / G free
    if (c + 1 < nch) load_a(c + 1);
    cp_async_commit();
    if (w < 4) {   // S <- e^{G_end} S + K^T U'
      const float eend = __expf(Gend);
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
        for (int n = 0; n < 4; ++n) { S[mi][n][0] *= eend; S[mi][n][1] *= eend; S[mi][n][2] *= eend; S[mi][n][3] *= eend; }
        warp_gemm<4, 8, true, false>(S[mi], Ksm + 32 * w + 16 * mi, kLdX, Upsm, kLdS);
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const int row = 32 * w + 16 * mi + g, col = 8 * n + 2 * tq;
          *reinterpret_cast<float2*>(Sop + row * kLdS + col) = make_float2(tf32r(S[mi][n][0]), tf32r(S[mi][n][1]));
          *reinterpret_cast<float2*>(Sop + (row + 8) * kLdS + col) = make_float2(tf32r(S[mi][n][2]), tf32r(S[mi][n][3]));
        }
      }
    } else {       // readout part 2: + QKd U, then store
      warp_gemm<4, 8, false, false>(acc, QKsm + mt * 16 * kLdM, kLdM, Usm, kLdS);
      const int r_lo = c * kChunk + mt * 16 + g, r_hi = r_lo + 8;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = h * 128 + col0 + 8 * n + 2 * tq;
        if (r_lo < R) *reinterpret_cast<float2*>(P.yraw + (size_t)r_lo * VW + col) = make_float2(acc[n][0], acc[n][1]);
        if (r_hi < R) *reinterpret_cast<float2*>(P.yraw + (size_t)r_hi * VW + col) = make_float2(acc[n][2], acc[n][3]);
      }
    }
    // the barrier at the top of the next iteration orders: S operand written / K, QKd, U, U' free
  }
  cp_async_wait_all();
  if (w < 4) {
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int row = 32 * w + 16 * mi + g, col = 8 * n + 2 * tq;
        *reinterpret_cast<float2*>(st + (size_t)row * 128 + col) = make_float2(S[mi][n][0], S[mi][n][1]);
        *reinterpret_cast<float2*>(st + (size_t)(row + 8) * 128 + col) = make_float2(S[mi][n][2], S[mi][n][3]);
      }
  }
}

bool gdn_chunk_available() { return true; }

static size_t chunk_layout(const cr_geometry* g, int rows, ChunkWs* ws, char* base) {
  const size_t chunks = (size_t)(rows + kChunk - 1) / kChunk, Hv = g->gdn_vheads;
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
  const size_t oW = take(Hv * chunks * 64 * 128 * 4), oU = take(Hv * chunks * 64 * 128 * 4);
  const size_t oQ = take(Hv * chunks * 64 * 64 * 4), oG = take(Hv * chunks * 64 * 4);
  if (ws) {
    ws->W = (float*)(base + oW); ws->Ut = (float*)(base + oU); ws->QKd = (float*)(base + oQ); ws->G = (float*)(base + oG);
    ws->chunks = (int)chunks;
  }
  return off;
}

size_t gdn_chunk_workspace_bytes(const cr_geometry* g, int rows) { return chunk_layout(g, rows, nullptr, nullptr); }

cr_status gdn_chunk_scan(const cr_geometry* g, const GdnPrefillParams& P, cudaStream_t stream) {
  ChunkWs ws;
  chunk_layout(g, P.a.R, &ws, P.chunk_ws);
  static bool configured = false;
  if (!configured) {
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLocalSmem));
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScanSmem));
    configured = true;
  }
  gdn_chunk_local_kernel<<<dim3(ws.chunks, g->gdn_kheads), 256, kLocalSmem, stream>>>(P, ws);
  CR_LAUNCH_CHECK("gdn_chunk_local_kernel");
  gdn_chunk_scan_kernel<<<g->gdn_vheads * 4, 256, kScanSmem, stream>>>(P, ws);
  CR_LAUNCH_CHECK("gdn_chunk_scan_kernel");
  return CR_OK;
}

}  // namespace cr
