// gdn_chunk_local_kernel: everything of the chunk-64 WY scan that does not depend on the carried state, fully
// parallel over (chunk, key head).  It reads the raw projection rows directly: conv(4) + SiLU + L2 norm of the
// key head's q and k (written once for the scan), the Gram matrices K K^T and Q K^T on tensor cores (kept in
// accumulator registers and shared by the value heads of the key head), and per value head: the log-decay
// prefix, L, the exact fp32 blocked inverse T = (I + L)^-1 (in place), W = T (beta e^G K), Ut = T (beta V) and QKd.
// Two CTAs fit per SM (92 KB of shared memory each), so one CTA's loads hide behind the other's math.
#include "gdn_chunk.cuh"

namespace cr {

constexpr size_t kLocalSmem = (size_t)(64 * kLdK + 64 * kLdX + 64 * kLdM + 16 * 64 + 3 * 64 + 64 * 4) * sizeof(float);

// Raw projection value pair (channels ch, ch+1; ch even) at call row r: this call's rows, the ring for rows
// before it, zero before position 0 and past the last row.
template <bool BF16>
__device__ __forceinline__ float2 raw_pair(const cr_gdn_args& a, int C, int r, int ch) {
  if (r >= a.R) return make_float2(0.f, 0.f);
  if (r >= 0) {
    if constexpr (BF16) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const __nv_bfloat16*>(a.qkv) + (size_t)r * C + ch);
      return __bfloat1622float2(v);
    } else {
      return *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(a.qkv) + (size_t)r * C + ch);
    }
  }
  const int p = a.pos0 + r;
  if (p < 0) return make_float2(0.f, 0.f);
  return *reinterpret_cast<const float2*>(a.hist + (size_t)(p & 15) * C + ch);
}

// conv(4) + SiLU of channels ch, ch+1 over ROWS consecutive rows starting at call row row0; out(i, value pair).
template <bool BF16, int ROWS, typename F>
__device__ __forceinline__ void conv_rows(const cr_gdn_args& a, int C, int row0, int ch, F&& out) {
  const float4 w0 = *reinterpret_cast<const float4*>(a.conv + (size_t)ch * 4);
  const float4 w1 = *reinterpret_cast<const float4*>(a.conv + (size_t)(ch + 1) * 4);
  float2 x0 = raw_pair<BF16>(a, C, row0 - 3, ch), x1 = raw_pair<BF16>(a, C, row0 - 2, ch), x2 = raw_pair<BF16>(a, C, row0 - 1, ch);
#pragma unroll 4
  for (int i = 0; i < ROWS; ++i) {
    const float2 x3 = raw_pair<BF16>(a, C, row0 + i, ch);
    float c0 = w0.x * x0.x, c1 = w1.x * x0.y;
    c0 = fmaf(w0.y, x1.x, c0); c1 = fmaf(w1.y, x1.y, c1);
    c0 = fmaf(w0.z, x2.x, c0); c1 = fmaf(w1.z, x2.y, c1);
    c0 = fmaf(w0.w, x3.x, c0); c1 = fmaf(w1.w, x3.y, c1);
    const bool live = row0 + i < a.R;
    out(i, make_float2(live ? siluf_(c0) : 0.f, live ? siluf_(c1) : 0.f));
    x0 = x1; x1 = x2; x2 = x3;
  }
}

// UM: operands for the tcgen05 scan are written as K-major tiles float[K/4][rows][4] (plus Qt = e^G Q and K^T).
template <bool BF16, bool UM>
__global__ void __launch_bounds__(256, 2) gdn_chunk_local_kernel(GdnPrefillParams P, ChunkWs ws) {
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm;                       // [64][132] khat (tf32)
  float* Qx = Ks + 64 * kLdK;           // [64][132] qhat, later [64][136] X = beta e^G K / beta V
  float* LT = Qx + 64 * kLdX;           // [64][68]  L, inverted in place to T
  float* Ms = LT + 64 * kLdM;           // [16][64]  scratch of the blocked inverse
  float* Gs = Ms + 16 * 64;             // [64] cumulative log decay
  float* bs = Gs + 64;                  // [64] beta
  float* es = bs + 64;                  // [64] beta * exp(G)
  float* red = es + 64;                 // [64][4] partial sums of squares: q halves, k halves
  const cr_gdn_args& a = P.a;
  const int c = blockIdx.x, kh = blockIdx.y;
  const int t = threadIdx.x, w = t >> 5, l = t & 31, g = l >> 2, tq = l & 3;
  const int R = a.R, r0 = c * kChunk, valid = min(kChunk, R - r0);
  const int rep = P.Hv / P.Hk, KW = P.Hk * 128, VW = P.Hv * 128, C = 2 * KW + VW;

  {   // q and k of the key head: conv + SiLU into shared memory, sums of squares per row
    const int part = (t >> 6) & 1, half = t >> 7, cp = t & 63;
    float* dst = part ? Ks : Qx;
    conv_rows<BF16, 32>(a, C, r0 + 32 * half, (part ? KW : 0) + kh * 128 + 2 * cp, [&](int i, float2 v) {
      const int row = 32 * half + i;
      *reinterpret_cast<float2*>(dst + row * kLdK + 2 * cp) = v;
      const float s = warp_sum(v.x * v.x + v.y * v.y);
      if (l == 0) red[row * 4 + part * 2 + (w & 1)] = s;
    });
  }
  __syncthreads();
  for (int i = t; i < 64 * 32; i += 256) {   // normalise, round to tf32, publish for the scan
    const int row = i >> 5, c4 = (i & 31) * 4;
    const float sq = rsqrtf(red[row * 4] + red[row * 4 + 1] + kEps) * kInvSqrt128;
    const float sk = rsqrtf(red[row * 4 + 2] + red[row * 4 + 3] + kEps);
    float4 q = *reinterpret_cast<float4*>(Qx + row * kLdK + c4), k = *reinterpret_cast<float4*>(Ks + row * kLdK + c4);
    q = make_float4(tf32r(q.x * sq), tf32r(q.y * sq), tf32r(q.z * sq), tf32r(q.w * sq));
    k = make_float4(tf32r(k.x * sk), tf32r(k.y * sk), tf32r(k.z * sk), tf32r(k.w * sk));
    *reinterpret_cast<float4*>(Qx + row * kLdK + c4) = q;
    *reinterpret_cast<float4*>(Ks + row * kLdK + c4) = k;
    if (row < valid) {
      *reinterpret_cast<float4*>(P.qn + ((size_t)(r0 + row) * P.Hk + kh) * 128 + c4) = q;
      *reinterpret_cast<float4*>(P.kn + ((size_t)(r0 + row) * P.Hk + kh) * 128 + c4) = k;
    }
  }
  __syncthreads();
  if constexpr (UM) {   // K^T of the chunk, K-major over tokens: unit (token/4, key) holds 4 tokens of one key
    float* kt = ws.Kt + ((size_t)kh * ws.chunks + c) * 8192;
    for (int i = t; i < 16 * 128; i += 256) {
      const int key = i & 127, tc = i >> 7;
      *reinterpret_cast<float4*>(kt + (size_t)i * 4) = make_float4(Ks[(4 * tc) * kLdK + key], Ks[(4 * tc + 1) * kLdK + key],
                                                                   Ks[(4 * tc + 2) * kLdK + key], Ks[(4 * tc + 3) * kLdK + key]);
    }
  }
  // Gram matrices stay in registers: warps 0-3 hold K K^T, warps 4-7 hold Q K^T, 16 rows each
  const int mt = w & 3, nh = w >> 2;
  float gram[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) gram[n][0] = gram[n][1] = gram[n][2] = gram[n][3] = 0.f;
  warp_gemm<8, 16, false, true>(gram, (w < 4 ? Ks : Qx) + mt * 16 * kLdK, kLdK, Ks, kLdK);
  __syncthreads();                       // qhat is no longer read from Qx

  for (int vi = 0; vi < rep; ++vi) {
    const int h = kh * rep + vi;
    const size_t unit = (size_t)h * ws.chunks + c;
    if (w == 0) {   // g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b); prefix sum (padding rows: 0)
      const float A = -expf(a.A_log[h]), dtb = a.dt_bias[h];
      float gv[2], bv[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int i = 2 * l + k;
        gv[k] = 0.f; bv[k] = 0.f;
        if (i < valid) {
          const float sp = load_in<BF16>(P.ab_logits, (size_t)(r0 + i) * 2 * P.Hv + h) + dtb;
          gv[k] = A * (sp > 20.f ? sp : log1pf(expf(sp)));
          bv[k] = sigmoidf_(load_in<BF16>(P.ab_logits, (size_t)(r0 + i) * 2 * P.Hv + P.Hv + h));
        }
      }
      float s = gv[0] + gv[1];
#pragma unroll
      for (int step = 1; step < 32; step <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, s, step);
        if (l >= step) s += v;
      }
      const float G1 = s, G0 = s - gv[1];
      Gs[2 * l] = G0; Gs[2 * l + 1] = G1; bs[2 * l] = bv[0]; bs[2 * l + 1] = bv[1];
      es[2 * l] = bv[0] * __expf(G0); es[2 * l + 1] = bv[1] * __expf(G1);
      ws.G[unit * 64 + 2 * l] = G0; ws.G[unit * 64 + 2 * l + 1] = G1;
    }
    __syncthreads();
    {   // L (warps 0-3) and QKd (warps 4-7) straight from the Gram fragments
      float* qkd = ws.QKd + unit * 64 * 64;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
          const int row = mt * 16 + g + 8 * hrow, col = n * 8 + 2 * tq;
          const float Gr = Gs[row];
          const float p0 = __expf(fminf(Gr - Gs[col], 0.f)), p1 = __expf(fminf(Gr - Gs[col + 1], 0.f));
          const float v0 = gram[n][2 * hrow], v1 = gram[n][2 * hrow + 1];
          if (w < 4) {
            const float b = bs[row];
            *reinterpret_cast<float2*>(LT + row * kLdM + col) = make_float2(col < row ? b * v0 * p0 : 0.f, col + 1 < row ? b * v1 * p1 : 0.f);
          } else {
            const int at = UM ? ((col >> 2) * 64 + row) * 4 + (col & 3) : row * 64 + col;
            *reinterpret_cast<float2*>(qkd + at) = make_float2(col <= row ? tf32r(v0 * p0) : 0.f, col + 1 <= row ? tf32r(v1 * p1) : 0.f);
          }
        }
    }
    for (int i = t; i < 64 * 32; i += 256) {   // X = beta e^G K
      const int row = i >> 5, c4 = (i & 31) * 4;
      const float4 kv = *reinterpret_cast<const float4*>(Ks + row * kLdK + c4);
      const float e = es[row];
      *reinterpret_cast<float4*>(Qx + row * kLdX + c4) = make_float4(tf32r(e * kv.x), tf32r(e * kv.y), tf32r(e * kv.z), tf32r(e * kv.w));
    }
    if constexpr (UM) {   // Qt = e^G Q of this value head, K-major over keys (q was published to qn above)
      float* qt = ws.Qt + unit * 8192;
      for (int i = t; i < 32 * 64; i += 256) {
        const int row = i & 63, kc = i >> 6;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < valid) q = *reinterpret_cast<const float4*>(P.qn + ((size_t)(r0 + row) * P.Hk + kh) * 128 + kc * 4);
        const float e = __expf(Gs[row]);
        *reinterpret_cast<float4*>(qt + (size_t)i * 4) = make_float4(tf32r(e * q.x), tf32r(e * q.y), tf32r(e * q.z), tf32r(e * q.w));
      }
    }
    __syncthreads();
    // T = (I + L)^-1 in exact fp32, blocked 16x16, in place.  Diagonal blocks: forward substitution, one thread
    // per column with the column in registers.  Block row a below the diagonal: T_a = -T_aa (L_a T_above).
    float D[16];
    if (t < 64) {
      const int b = t >> 4, j = t & 15;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = (i == j) ? 1.f : 0.f;
#pragma unroll
        for (int m = 0; m < i; ++m) acc = fmaf(-LT[(16 * b + i) * kLdM + 16 * b + m], D[m], acc);
        D[i] = acc;
      }
    }
    __syncthreads();
    if (t < 64) {
      const int b = t >> 4, j = t & 15;
#pragma unroll
      for (int i = 0; i < 16; ++i) LT[(16 * b + i) * kLdM + 16 * b + j] = D[i];
    }
    __syncthreads();
    for (int ab = 1; ab < 4; ++ab) {
      const int wid = 16 * ab;
      for (int e = t; e < 16 * wid; e += 256) {  // M = L_a T_above
        const int i = e / wid, j = e % wid;
        float acc = 0.f;
        for (int m = j & ~15; m < wid; ++m) acc = fmaf(LT[(wid + i) * kLdM + m], LT[m * kLdM + j], acc);
        Ms[i * 64 + j] = acc;
      }
      __syncthreads();
      for (int e = t; e < 16 * wid; e += 256) {  // T_a = -T_aa M
        const int i = e / wid, j = e % wid;
        float acc = 0.f;
        for (int m = 0; m <= i; ++m) acc = fmaf(LT[(wid + i) * kLdM + wid + m], Ms[m * 64 + j], acc);
        LT[(wid + i) * kLdM + j] = -acc;
      }
      __syncthreads();
    }
    for (int i = t; i < 64 * 64; i += 256) {
      float* p = LT + (i >> 6) * kLdM + (i & 63);
      *p = tf32r(*p);
    }
    __syncthreads();
    {   // W = T X
      float acc[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      warp_gemm<8, 8, false, false>(acc, LT + mt * 16 * kLdM, kLdM, Qx + nh * 64, kLdX);
      if constexpr (UM) {
        float* dst = ws.W + unit * 8192;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const int col = nh * 64 + n * 8 + 2 * tq, r_lo = mt * 16 + g;
          *reinterpret_cast<float2*>(dst + ((col >> 2) * 64 + r_lo) * 4 + (col & 3)) = make_float2(tf32r(acc[n][0]), tf32r(acc[n][1]));
          *reinterpret_cast<float2*>(dst + ((col >> 2) * 64 + r_lo + 8) * 4 + (col & 3)) = make_float2(tf32r(acc[n][2]), tf32r(acc[n][3]));
        }
      } else {
        float* dst = ws.W + (unit * 64 + mt * 16) * 128 + nh * 64;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          *reinterpret_cast<float2*>(dst + g * 128 + n * 8 + 2 * tq) = make_float2(tf32r(acc[n][0]), tf32r(acc[n][1]));
          *reinterpret_cast<float2*>(dst + (g + 8) * 128 + n * 8 + 2 * tq) = make_float2(tf32r(acc[n][2]), tf32r(acc[n][3]));
        }
      }
    }
    __syncthreads();
    {   // X = beta SiLU(conv(v)) of value head h
      const int quarter = t >> 6, cp = t & 63;
      conv_rows<BF16, 16>(a, C, r0 + 16 * quarter, 2 * KW + h * 128 + 2 * cp, [&](int i, float2 v) {
        const int row = 16 * quarter + i;
        const float b = bs[row];
        *reinterpret_cast<float2*>(Qx + row * kLdX + 2 * cp) = make_float2(tf32r(b * v.x), tf32r(b * v.y));
      });
    }
    __syncthreads();
    {   // Ut = T X  (fp32: it is added, not multiplied, in the scan)
      float acc[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      warp_gemm<8, 8, false, false>(acc, LT + mt * 16 * kLdM, kLdM, Qx + nh * 64, kLdX);
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
