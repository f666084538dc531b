// gdn_chunk_local_kernel: everything of the chunk-64 WY scan that does not depend on the carried state, fully
// parallel over (chunk, key head).  Per CTA:
//   1. raw projection rows of the key head's q and k channels are staged in shared memory with 128-bit loads
//      (3 halo rows from the previous rows, the ring, or zero), then conv(4) + SiLU + L2 norm -> qhat, khat (tf32);
//   2. Gram matrices K K^T and Q K^T on tensor cores, kept in accumulator registers for all value heads;
//   3. per value head: log-decay prefix G and beta, L = tril(beta K K^T e^{dG}, -1), QKd = tril(Q K^T e^{dG}), and
//      W = (I + L)^-1 (beta e^G K),  Ut = (I + L)^-1 (beta V)  by exact fp32 forward substitution: one thread per
//      output column with the column in registers, L rows broadcast from shared memory, no barriers; the v
//      columns run conv + SiLU on the fly from the staged raw rows.
// Outputs go straight into the layouts the scan consumes (K-major tiles for the tcgen05 scan).
// Two CTAs fit per SM (106 KB of shared memory each), so one CTA's loads hide behind the other's math.
#include "gdn_chunk.cuh"

namespace cr {

constexpr int kRawRows = 67;                               // 64 rows + 3 halo rows
constexpr int kStageBytes = kRawRows * 128 * 2;            // one 128-channel bf16 tile (or 64 fp32 channels)
constexpr size_t kLocalSmem = (size_t)(2 * 64 * kLdK + 64 * kLdM + 9 * 64 + 64 * 4) * sizeof(float) + kStageBytes + 256;

// Stages rows row0-3 .. row0+63 of channels [ch0, ch0+CH) into dst[67][CH] (element type of the input).
// Rows before the call come from the input itself (halo_in: a later part of one call), the ring, or zero.
template <bool BF16, int CH>
__device__ __forceinline__ void stage_raw(const GdnPrefillParams& P, int C, int row0, int ch0, void* dst) {
  constexpr int EPV = BF16 ? 8 : 4;                        // elements per 16-byte piece
  constexpr int PPR = CH / EPV;                            // pieces per row
  const cr_gdn_args& a = P.a;
  for (int i = threadIdx.x; i < kRawRows * PPR; i += 256) {
    const int rr = i / PPR, pc = i % PPR, r = row0 - 3 + rr, ch = ch0 + pc * EPV;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < a.R) {
      if (r >= 0 || P.halo_in) {
        v = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(a.qkv) + ((long long)r * C + ch) * (BF16 ? 2 : 4));
      } else if (a.pos0 + r >= 0) {
        const float* hs = a.hist + (size_t)((a.pos0 + r) & 15) * C + ch;
        if constexpr (BF16) {
          __nv_bfloat162 b[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) b[k] = __floats2bfloat162_rn(hs[2 * k], hs[2 * k + 1]);
          v = *reinterpret_cast<const uint4*>(b);
        } else {
          v = *reinterpret_cast<const uint4*>(hs);
        }
      }
    }
    reinterpret_cast<uint4*>(dst)[i] = v;
  }
}
template <bool BF16>
__device__ __forceinline__ float2 staged_pair(const void* buf, int CH, int rr, int ch) {
  if constexpr (BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const __nv_bfloat16*>(buf) + rr * CH + ch));
  else return *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(buf) + rr * CH + ch);
}
template <bool BF16>
__device__ __forceinline__ float staged_one(const void* buf, int CH, int rr, int ch) {
  if constexpr (BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(buf)[rr * CH + ch]);
  else return reinterpret_cast<const float*>(buf)[rr * CH + ch];
}

// out[i] = x(i) - sum_{m<i} L[i][m] out[m] for i < 64: the thread's column of (I + L)^-1 X, exact fp32.
template <typename FX, typename FO>
__device__ __forceinline__ void solve_column(const float* LT, FX&& x, FO&& emit) {
  float out[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    float a0 = x(i), a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int m4 = 0; m4 < (i + 3) / 4; ++m4) {
      const float4 lv = *reinterpret_cast<const float4*>(&LT[i * kLdM + m4 * 4]);
      a0 = fmaf(-lv.x, out[m4 * 4], a0);
      if (m4 * 4 + 1 < i) a1 = fmaf(-lv.y, out[m4 * 4 + 1], a1);
      if (m4 * 4 + 2 < i) a2 = fmaf(-lv.z, out[m4 * 4 + 2], a2);
      if (m4 * 4 + 3 < i) a3 = fmaf(-lv.w, out[m4 * 4 + 3], a3);
    }
    out[i] = (a0 + a1) + (a2 + a3);
    emit(i, out[i]);
  }
}

// UM: operands for the tcgen05 scan are written as K-major tiles float[K/4][rows][4] (plus Qt = e^G Q and K^T);
// otherwise row-major tiles and the prepared q/k rows for the mma.sync scan.
template <bool BF16, bool UM>
__global__ void __launch_bounds__(256, 2) gdn_chunk_local_kernel(GdnPrefillParams P, ChunkWs ws) {
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm;                       // [64][132] khat (tf32)
  float* Qs = Ks + 64 * kLdK;           // [64][132] qhat (tf32); with fp32 inputs later the head of the v staging tile
  char* RB = reinterpret_cast<char*>(Qs + 64 * kLdK);      // raw staging tile (directly after Qs)
  float* LT = reinterpret_cast<float*>(RB + kStageBytes);  // [64][68] L
  float* Gs = LT + 64 * kLdM;           // [3][64] cumulative log decay per value head
  float* bs = Gs + 3 * 64;              // [3][64] beta
  float* es = bs + 3 * 64;              // [3][64] beta * exp(G)
  float* red = es + 3 * 64;             // [64][4] partial sums of squares: q halves, k halves
  const cr_gdn_args& a = P.a;
  const int c = blockIdx.x, kh = blockIdx.y;
  const int t = threadIdx.x, w = t >> 5, l = t & 31, g = l >> 2, tq = l & 3;
  const int R = a.R, r0 = c * kChunk, valid = min(kChunk, R - r0);
  const int rep = P.Hv / P.Hk, KW = P.Hk * 128, VW = P.Hv * 128, C = 2 * KW + VW;
  constexpr int CH = BF16 ? 128 : 64;   // channels per staging round
  constexpr int PAIRS = CH / 2, RSEG = 256 / PAIRS, RPT = 64 / RSEG;

  // ---- 1. q and k of the key head
  for (int part = 0; part < 2; ++part) {
    float* dst = part ? Ks : Qs;
    for (int round = 0; round < 128 / CH; ++round) {
      __syncthreads();                  // staging tile free
      stage_raw<BF16, CH>(P, C, r0, (part ? KW : 0) + kh * 128 + round * CH, RB);
      __syncthreads();
      const int cp = t % PAIRS, seg = t / PAIRS, chl = 2 * cp, chg = (part ? KW : 0) + kh * 128 + round * CH + chl;
      const float4 w0 = *reinterpret_cast<const float4*>(a.conv + (size_t)chg * 4);
      const float4 w1 = *reinterpret_cast<const float4*>(a.conv + (size_t)(chg + 1) * 4);
      const int rb = seg * RPT;         // first chunk row of this thread; staged row index = chunk row + 3
      float2 x0 = staged_pair<BF16>(RB, CH, rb, chl), x1 = staged_pair<BF16>(RB, CH, rb + 1, chl), x2 = staged_pair<BF16>(RB, CH, rb + 2, chl);
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const float2 x3 = staged_pair<BF16>(RB, CH, rb + 3 + i, chl);
        float c0 = w0.x * x0.x, c1 = w1.x * x0.y;
        c0 = fmaf(w0.y, x1.x, c0); c1 = fmaf(w1.y, x1.y, c1);
        c0 = fmaf(w0.z, x2.x, c0); c1 = fmaf(w1.z, x2.y, c1);
        c0 = fmaf(w0.w, x3.x, c0); c1 = fmaf(w1.w, x3.y, c1);
        const bool live = rb + i < valid;
        const float v0 = live ? siluf_(c0) : 0.f, v1 = live ? siluf_(c1) : 0.f;
        *reinterpret_cast<float2*>(dst + (rb + i) * kLdK + round * CH + chl) = make_float2(v0, v1);
        const float s = warp_sum(v0 * v0 + v1 * v1);     // a warp covers 64 channels of one row
        if (l == 0) red[(rb + i) * 4 + part * 2 + (BF16 ? (w & 1) : round)] = s;
        x0 = x1; x1 = x2; x2 = x3;
      }
    }
  }
  __syncthreads();
  for (int i = t; i < 64 * 32; i += 256) {   // normalise and round to tf32
    const int row = i >> 5, c4 = (i & 31) * 4;
    const float sq = rsqrtf(red[row * 4] + red[row * 4 + 1] + kEps) * kInvSqrt128;
    const float sk = rsqrtf(red[row * 4 + 2] + red[row * 4 + 3] + kEps);
    float4 q = *reinterpret_cast<float4*>(Qs + row * kLdK + c4), k = *reinterpret_cast<float4*>(Ks + row * kLdK + c4);
    q = make_float4(tf32r(q.x * sq), tf32r(q.y * sq), tf32r(q.z * sq), tf32r(q.w * sq));
    k = make_float4(tf32r(k.x * sk), tf32r(k.y * sk), tf32r(k.z * sk), tf32r(k.w * sk));
    *reinterpret_cast<float4*>(Qs + row * kLdK + c4) = q;
    *reinterpret_cast<float4*>(Ks + row * kLdK + c4) = k;
    if (!UM && row < valid) {
      *reinterpret_cast<float4*>(P.qn + ((size_t)(r0 + row) * P.Hk + kh) * 128 + c4) = q;
      *reinterpret_cast<float4*>(P.kn + ((size_t)(r0 + row) * P.Hk + kh) * 128 + c4) = k;
    }
  }
  if (w < rep) {   // g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b); prefix sum; one warp per value head
    const int h = kh * rep + w;
    const float A = -expf(a.A_log[h]), dtb = a.dt_bias[h];
    float gv[2], bv[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = 2 * l + k;
      gv[k] = 0.f; bv[k] = 0.f;
      if (i < valid) {
        const float sp = load_in<BF16>(P.ab_logits, (long long)(r0 + i) * 2 * P.Hv + h) + dtb;
        gv[k] = A * (sp > 20.f ? sp : log1pf(expf(sp)));
        bv[k] = sigmoidf_(load_in<BF16>(P.ab_logits, (long long)(r0 + i) * 2 * P.Hv + P.Hv + h));
      }
    }
    float s = gv[0] + gv[1];
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, s, step);
      if (l >= step) s += v;
    }
    const float G1 = s, G0 = s - gv[1];
    float* Gw = Gs + w * 64; float* bw = bs + w * 64; float* ew = es + w * 64;
    Gw[2 * l] = G0; Gw[2 * l + 1] = G1; bw[2 * l] = bv[0]; bw[2 * l + 1] = bv[1];
    ew[2 * l] = bv[0] * __expf(G0); ew[2 * l + 1] = bv[1] * __expf(G1);
    float* Gg = ws.G + ((size_t)h * ws.chunks + c) * 64;
    Gg[2 * l] = G0; Gg[2 * l + 1] = G1;
  }
  __syncthreads();
  if constexpr (UM) {
    // K^T of the chunk, K-major over tokens: unit (token/4, key) holds 4 tokens of one key
    float* kt = ws.Kt + ((size_t)kh * ws.chunks + c) * 8192;
    for (int i = t; i < 16 * 128; i += 256) {
      const int key = i & 127, tc = i >> 7;
      *reinterpret_cast<float4*>(kt + (size_t)i * 4) = make_float4(Ks[(4 * tc) * kLdK + key], Ks[(4 * tc + 1) * kLdK + key],
                                                                   Ks[(4 * tc + 2) * kLdK + key], Ks[(4 * tc + 3) * kLdK + key]);
    }
    // Qt = e^G Q per value head, K-major over keys
    for (int vi = 0; vi < rep; ++vi) {
      float* qt = ws.Qt + ((size_t)(kh * rep + vi) * ws.chunks + c) * 8192;
      for (int i = t; i < 32 * 64; i += 256) {
        const int row = i & 63, kc = i >> 6;
        const float4 q = *reinterpret_cast<const float4*>(Qs + row * kLdK + kc * 4);
        const float e = __expf(Gs[vi * 64 + row]);
        *reinterpret_cast<float4*>(qt + (size_t)i * 4) = make_float4(tf32r(e * q.x), tf32r(e * q.y), tf32r(e * q.z), tf32r(e * q.w));
      }
    }
  }
  // ---- 2. Gram matrices stay in registers: warps 0-3 hold K K^T, warps 4-7 hold Q K^T, 16 rows each
  const int mt = w & 3;
  float gram[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) gram[n][0] = gram[n][1] = gram[n][2] = gram[n][3] = 0.f;
  warp_gemm<8, 16, false, true>(gram, (w < 4 ? Ks : Qs) + mt * 16 * kLdK, kLdK, Ks, kLdK);

  // ---- 3. per value head
  for (int vi = 0; vi < rep; ++vi) {
    const int h = kh * rep + vi;
    const size_t unit = (size_t)h * ws.chunks + c;
    const float* Gv = Gs + vi * 64; const float* bv = bs + vi * 64; const float* ev = es + vi * 64;
    __syncthreads();                    // previous head done with LT and the staging tile; qhat no longer needed
    {   // L (warps 0-3) and QKd (warps 4-7) straight from the Gram fragments
      float* qkd = ws.QKd + unit * 64 * 64;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
          const int row = mt * 16 + g + 8 * hrow, col = n * 8 + 2 * tq;
          const float Gr = Gv[row];
          const float p0 = __expf(fminf(Gr - Gv[col], 0.f)), p1 = __expf(fminf(Gr - Gv[col + 1], 0.f));
          const float v0 = gram[n][2 * hrow], v1 = gram[n][2 * hrow + 1];
          if (w < 4) {
            const float b = bv[row];
            *reinterpret_cast<float2*>(LT + row * kLdM + col) = make_float2(col < row ? b * v0 * p0 : 0.f, col + 1 < row ? b * v1 * p1 : 0.f);
          } else {
            const int at = UM ? ((col >> 2) * 64 + row) * 4 + (col & 3) : row * 64 + col;
            *reinterpret_cast<float2*>(qkd + at) = make_float2(col <= row ? tf32r(v0 * p0) : 0.f, col + 1 <= row ? tf32r(v1 * p1) : 0.f);
          }
        }
    }
    // raw v rows of value head h: 128 channels (with fp32 inputs the tile spills into the freed qhat buffer)
    void* vbuf = BF16 ? (void*)RB : (void*)Qs;
    stage_raw<BF16, 128>(P, C, r0, 2 * KW + h * 128, vbuf);
    __syncthreads();
    if (t < 128) {   // W column (key t): X = beta e^G K
      float* Wg = ws.W + unit * 8192;
      solve_column(LT, [&](int i) { return ev[i] * Ks[i * kLdK + t]; },
                   [&](int i, float v) { Wg[UM ? ((t >> 2) * 64 + i) * 4 + (t & 3) : i * 128 + t] = tf32r(v); });
    } else {         // Ut column (value channel t - 128): X = beta SiLU(conv(v)), conv fused into the recurrence
      const int d = t - 128;
      const float4 wv = *reinterpret_cast<const float4*>(a.conv + (size_t)(2 * KW + h * 128 + d) * 4);
      float x0 = staged_one<BF16>(vbuf, 128, 0, d), x1 = staged_one<BF16>(vbuf, 128, 1, d), x2 = staged_one<BF16>(vbuf, 128, 2, d);
      float* Ug = ws.Ut + unit * 8192 + d;
      solve_column(LT,
                   [&](int i) {
                     const float x3 = staged_one<BF16>(vbuf, 128, i + 3, d);
                     float cv = wv.x * x0;
                     cv = fmaf(wv.y, x1, cv); cv = fmaf(wv.z, x2, cv); cv = fmaf(wv.w, x3, cv);
                     x0 = x1; x1 = x2; x2 = x3;
                     return i < valid ? bv[i] * siluf_(cv) : 0.f;
                   },
                   [&](int i, float v) { Ug[i * 128] = v; });
    }
  }
}

cr_status gdn_chunk_local_launch(const cr_geometry* g, const GdnPrefillParams& P, const ChunkWs& ws, bool bf16_in, bool umma_layout,
                                 cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_local_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLocalSmem));
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_local_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLocalSmem));
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_local_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLocalSmem));
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_local_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLocalSmem));
    configured = true;
  }
  const dim3 grid(ws.chunks, g->gdn_kheads);
  if (bf16_in && umma_layout) gdn_chunk_local_kernel<true, true><<<grid, 256, kLocalSmem, stream>>>(P, ws);
  else if (bf16_in) gdn_chunk_local_kernel<true, false><<<grid, 256, kLocalSmem, stream>>>(P, ws);
  else if (umma_layout) gdn_chunk_local_kernel<false, true><<<grid, 256, kLocalSmem, stream>>>(P, ws);
  else gdn_chunk_local_kernel<false, false><<<grid, 256, kLocalSmem, stream>>>(P, ws);
  CR_LAUNCH_CHECK("gdn_chunk_local_kernel");
  return CR_OK;
}

}  // namespace cr
