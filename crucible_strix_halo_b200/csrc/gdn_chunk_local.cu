// gdn_chunk_local_kernel: everything of the chunk-64 WY scan that does not depend on the carried state, fully
// parallel over (chunk, key head).  Per CTA:
//   1. raw projection rows of the key head's q and k channels are staged in shared memory with cp.async (3 halo rows
//      from the previous rows, the ring, or zero; with bf16 inputs the next tile is always in flight while the
//      current one is used), then conv(4) + SiLU + L2 norm -> qhat, khat (tf32); the gates (log-decay prefix G, beta
//      and their exponential tables) of the value heads are computed while the first tiles arrive;
//   2. Gram matrices K K^T and Q K^T on tensor cores, kept in accumulator registers for all value heads;
//   3. per value head: K'^T = (e^{G_end - G} K)^T and e^G Q tiles, L = tril(beta K K^T e^{dG}, -1), QKd = tril(Q K^T e^{dG}), and
//      T = (I + L)^-1 by an exact fp32 blocked inverse (16 x 16 diagonal blocks by substitution, off-diagonal blocks
//      in block-row order), then W = T (beta e^G K) and Ut = T (beta V) on tensor cores with tf32 operands; the
//      v columns run conv + SiLU from the staged raw rows.
// Outputs go straight into the layouts the scan consumes (K-major tiles for the tcgen05 scan).
// Two CTAs fit per SM (110 KB of shared memory, 128 registers x 256 threads each), so one CTA's barriers and loads
// hide behind the other's math.
#include "gdn_chunk.cuh"

namespace cr {

constexpr int kRawRows = 67;                               // 64 rows + 3 halo rows
constexpr int kStageBytes = kRawRows * 128 * 2;            // one 128-channel bf16 tile (or 64 fp32 channels)
constexpr size_t kLocalSmem = (size_t)(64 * kLdK + 64 * kLdX + 64 * kLdM + 15 * 64 + 3 * 256) * sizeof(float) + kStageBytes + 256;

// Starts the copy of rows row0-3 .. row0+63 of channels [ch0, ch0+CH) into dst[67][CH] (element type of the input)
// as one cp.async group; rows past the end of the call are zero-filled.  Rows before the call come from the input
// itself (halo_in: a later part of one call), or, with plain stores, from the ring or zero.
template <bool BF16, int CH>
__device__ __forceinline__ void stage_issue(const GdnPrefillParams& P, int C, int row0, int ch0, void* dst) {
  constexpr int EPV = BF16 ? 8 : 4;                        // elements per 16-byte piece
  constexpr int PPR = CH / EPV;                            // pieces per row
  const cr_gdn_args& a = P.a;
  for (int i = threadIdx.x; i < kRawRows * PPR; i += 256) {
    const int rr = i / PPR, pc = i % PPR, r = row0 - 3 + rr, ch = ch0 + pc * EPV;
    uint4* d = reinterpret_cast<uint4*>(dst) + i;
    if (r >= 0 || P.halo_in) {
      const bool valid = r < a.R;
      cp_async16(d, reinterpret_cast<const char*>(a.qkv) + (valid ? ((long long)r * C + ch) * (BF16 ? 2 : 4) : 0ll), valid);
    } else {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (a.pos0 + r >= 0) {
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
      *d = v;
    }
  }
  cp_async_commit();
}
template <bool BF16, int CH>
__device__ __forceinline__ void stage_raw(const GdnPrefillParams& P, int C, int row0, int ch0, void* dst) {
  stage_issue<BF16, CH>(P, C, row0, ch0, dst);
  cp_async_wait_all();
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

// T = (I + L)^-1 for the 64x64 unit lower-triangular I + L held in LT, exact fp32, in place, by 16x16 blocks:
// diagonal blocks by forward substitution (one thread per column, column in registers), then block row by block
// row, T_ab = -T_aa (sum_{c=b}^{a-1} L_ac T_cb): every phase is a product of 16-long unrolled dot products with
// all 256 threads busy (thread = element (t/16, t%16) of each block of the row).
__device__ __forceinline__ void invert_unit_lower_64(float* LT, float* Ms) {
  const int t = threadIdx.x, i = t >> 4, j = t & 15;
  float D[16];
  if (t < 64) {
    const int b = t >> 4;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      float acc = (r == j) ? 1.f : 0.f;
#pragma unroll
      for (int m = 0; m < r; ++m) acc = fmaf(-LT[(16 * b + r) * kLdM + 16 * b + m], D[m], acc);
      D[r] = acc;
    }
  }
  __syncthreads();
  if (t < 64) {
    const int b = t >> 4;
#pragma unroll
    for (int r = 0; r < 16; ++r) LT[(16 * b + r) * kLdM + 16 * b + j] = D[r];
  }
  __syncthreads();
  for (int a = 1; a < 4; ++a) {          // block row a: its L blocks are still untouched
    float macc[3] = {0.f, 0.f, 0.f};     // M_ab = sum_{c=b}^{a-1} L_ac T_cb for b = 0 .. a-1; L_ac[i][m] is read once
#pragma unroll
    for (int cb = 0; cb < 3; ++cb) {
      if (cb < a) {
        const float* Lr = LT + (16 * a + i) * kLdM + 16 * cb;
#pragma unroll
        for (int m4 = 0; m4 < 16; m4 += 4) {
          const float4 lv = *reinterpret_cast<const float4*>(Lr + m4);
          const float lm[4] = {lv.x, lv.y, lv.z, lv.w};
#pragma unroll
          for (int mm = 0; mm < 4; ++mm) {
            const float* Tc = LT + (16 * cb + m4 + mm) * kLdM + j;
#pragma unroll
            for (int b = 0; b < 3; ++b)
              if (b <= cb) macc[b] = fmaf(lm[mm], Tc[16 * b], macc[b]);
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < 3; ++b)
      if (b < a) Ms[b * 256 + t] = macc[b];
    __syncthreads();
    {                                    // T_ab = -T_aa M_ab  (T_aa lower triangular: m <= i); the T_aa row is read once
      const float* Tr = LT + (16 * a + i) * kLdM + 16 * a;
      float tr[16];
#pragma unroll
      for (int m4 = 0; m4 < 16; m4 += 4) {
        const float4 v = *reinterpret_cast<const float4*>(Tr + m4);
        tr[m4] = m4 <= i ? v.x : 0.f; tr[m4 + 1] = m4 + 1 <= i ? v.y : 0.f;
        tr[m4 + 2] = m4 + 2 <= i ? v.z : 0.f; tr[m4 + 3] = m4 + 3 <= i ? v.w : 0.f;
      }
#pragma unroll
      for (int b = 0; b < 3; ++b) {
        if (b < a) {
          const float* Mc = Ms + b * 256 + j;
          float m0 = 0.f, m1 = 0.f;
#pragma unroll
          for (int m = 0; m < 16; m += 2) {
            m0 = fmaf(tr[m], Mc[m * 16], m0);
            m1 = fmaf(tr[m + 1], Mc[(m + 1) * 16], m1);
          }
          LT[(16 * a + i) * kLdM + 16 * b + j] = -(m0 + m1);
        }
      }
    }
    __syncthreads();
  }
}

// Operands for the tcgen05 scan are written as K-major tiles float[K/4][rows][4] (plus Qt = e^G Q and K'^T).
template <bool BF16>
__global__ void __launch_bounds__(256, 2) gdn_chunk_local_kernel(GdnPrefillParams P, ChunkWs ws) {
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm;                       // [64][132] khat (tf32)
  float* Qs = Ks + 64 * kLdK;           // [64][132] qhat (tf32), later [64][136] X = beta e^G K / beta V
  char* RB = reinterpret_cast<char*>(Qs + 64 * kLdX);      // raw staging tile
  float* LT = reinterpret_cast<float*>(RB + kStageBytes);  // [64][68] L
  float* Gs = LT + 64 * kLdM;           // [3][64] cumulative log decay per value head
  float* bs = Gs + 3 * 64;              // [3][64] beta
  float* es = bs + 3 * 64;              // [3][64] beta * exp(G)
  float* egs = es + 3 * 64;             // [3][64] exp(G)
  float* scs = egs + 3 * 64;            // [3][64] exp(G_end - G)
  float* Ms = scs + 3 * 64;             // [3][256] scratch of the blocked inverse
  const cr_gdn_args& a = P.a;
  const int c = blockIdx.x, kh = blockIdx.y;
  const int t = threadIdx.x, w = t >> 5, l = t & 31, g = l >> 2, tq = l & 3;
  const int R = a.R, r0 = c * kChunk, valid = min(kChunk, R - r0);
  const int rep = P.Hv / P.Hk, KW = P.Hk * 128, VW = P.Hv * 128, C = 2 * KW + VW;
  constexpr int CH = BF16 ? 128 : 64;   // channels per staging round
  constexpr int PAIRS = CH / 2, RSEG = 256 / PAIRS, RPT = 64 / RSEG;

  // ---- 1. q and k of the key head.  With bf16 inputs a whole 128-channel tile is one staging round: q goes to the
  // staging tile and k to the (still unused) L tile, both in flight at once; the first v tile follows as soon as
  // the staging tile is free, so its latency hides behind the Gram products.
  char* RB2 = reinterpret_cast<char*>(LT);
  if constexpr (BF16) {
    stage_issue<true, 128>(P, C, r0, kh * 128, RB);
    stage_issue<true, 128>(P, C, r0, KW + kh * 128, RB2);
  }
  // Gates while the first tiles are in flight: g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b), prefix sum of
  // g inside the chunk; one warp per value head.  The tables are read after later barriers.
  if (w < rep) {
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
    const float e0 = __expf(G0), e1 = __expf(G1), Gend = __shfl_sync(0xffffffffu, G1, 31);
    ew[2 * l] = bv[0] * e0; ew[2 * l + 1] = bv[1] * e1;
    egs[w * 64 + 2 * l] = e0; egs[w * 64 + 2 * l + 1] = e1;
    scs[w * 64 + 2 * l] = __expf(Gend - G0); scs[w * 64 + 2 * l + 1] = __expf(Gend - G1);
    float* Gg = ws.G + ((size_t)h * ws.chunks + c) * 64;
    Gg[2 * l] = G0; Gg[2 * l + 1] = G1;
  }
  for (int part = 0; part < 2; ++part) {
    float* dst = part ? Ks : Qs;
    for (int round = 0; round < 128 / CH; ++round) {
      const char* src = RB;
      if constexpr (BF16) {
        if (part == 0) cp_async_wait_but_one(); else cp_async_wait_all();
        __syncthreads();
        src = part ? RB2 : RB;
      } else {
        __syncthreads();                // staging tile free
        stage_raw<BF16, CH>(P, C, r0, (part ? KW : 0) + kh * 128 + round * CH, RB);
        __syncthreads();
      }
      const int cp = t % PAIRS, seg = t / PAIRS, chl = 2 * cp, chg = (part ? KW : 0) + kh * 128 + round * CH + chl;
      const float4 w0 = *reinterpret_cast<const float4*>(a.conv + (size_t)chg * 4);
      const float4 w1 = *reinterpret_cast<const float4*>(a.conv + (size_t)(chg + 1) * 4);
      const int rb = seg * RPT;         // first chunk row of this thread; staged row index = chunk row + 3
      float2 x0 = staged_pair<BF16>(src, CH, rb, chl), x1 = staged_pair<BF16>(src, CH, rb + 1, chl), x2 = staged_pair<BF16>(src, CH, rb + 2, chl);
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const float2 x3 = staged_pair<BF16>(src, CH, rb + 3 + i, chl);
        float c0 = w0.x * x0.x, c1 = w1.x * x0.y;
        c0 = fmaf(w0.y, x1.x, c0); c1 = fmaf(w1.y, x1.y, c1);
        c0 = fmaf(w0.z, x2.x, c0); c1 = fmaf(w1.z, x2.y, c1);
        c0 = fmaf(w0.w, x3.x, c0); c1 = fmaf(w1.w, x3.y, c1);
        const bool live = rb + i < valid;
        *reinterpret_cast<float2*>(dst + (rb + i) * kLdK + round * CH + chl) = make_float2(live ? siluf_(c0) : 0.f, live ? siluf_(c1) : 0.f);
        x0 = x1; x1 = x2; x2 = x3;
      }
    }
  }
  __syncthreads();
  if constexpr (BF16) stage_issue<true, 128>(P, C, r0, 2 * KW + kh * rep * 128, RB);   // v of the first value head
  for (int i = t; i < 64 * 32; i += 256) {   // L2 norms (a warp holds one row), scale, round to tf32
    const int row = i >> 5, c4 = (i & 31) * 4;
    float4 q = *reinterpret_cast<float4*>(Qs + row * kLdK + c4), k = *reinterpret_cast<float4*>(Ks + row * kLdK + c4);
    float sq = q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w, sk = k.x * k.x + k.y * k.y + k.z * k.z + k.w * k.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      sk += __shfl_xor_sync(0xffffffffu, sk, o);
    }
    sq = rsqrtf(sq + kEps) * kInvSqrt128;
    sk = rsqrtf(sk + kEps);
    q = make_float4(tf32r(q.x * sq), tf32r(q.y * sq), tf32r(q.z * sq), tf32r(q.w * sq));
    k = make_float4(tf32r(k.x * sk), tf32r(k.y * sk), tf32r(k.z * sk), tf32r(k.w * sk));
    *reinterpret_cast<float4*>(Qs + row * kLdK + c4) = q;
    *reinterpret_cast<float4*>(Ks + row * kLdK + c4) = k;
  }
  __syncthreads();
  {
    // per value head: K'^T = (e^{G_end - G} K)^T, K-major over tokens (unit (token / 4, key) holds 4 tokens of one
    // key; the decay towards the chunk end is folded into K so that the scan multiplies U itself), and
    // Qt = e^G Q, K-major over keys
    for (int vi = 0; vi < rep; ++vi) {
      float* kt = ws.Kt + ((size_t)(kh * rep + vi) * ws.chunks + c) * 8192;
      for (int i = t; i < 16 * 128; i += 256) {
        const int key = i & 127, tc = i >> 7;
        const float4 sc = *reinterpret_cast<const float4*>(scs + vi * 64 + 4 * tc);
        *reinterpret_cast<float4*>(kt + (size_t)i * 4) =
            make_float4(tf32r(sc.x * Ks[(4 * tc) * kLdK + key]), tf32r(sc.y * Ks[(4 * tc + 1) * kLdK + key]),
                        tf32r(sc.z * Ks[(4 * tc + 2) * kLdK + key]), tf32r(sc.w * Ks[(4 * tc + 3) * kLdK + key]));
      }
      float* qt = ws.WQ + ((size_t)(kh * rep + vi) * ws.chunks + c) * 16384;
      for (int i = t; i < 32 * 64; i += 256) {
        const int row = i & 63, kc = i >> 6;
        const float4 q = *reinterpret_cast<const float4*>(Qs + row * kLdK + kc * 4);
        const float e = egs[vi * 64 + row];
        *reinterpret_cast<float4*>(qt + (size_t)(kc * 128 + 64 + row) * 4) = make_float4(tf32r(e * q.x), tf32r(e * q.y), tf32r(e * q.z), tf32r(e * q.w));
      }
    }
  }
  // ---- 2. Gram matrices stay in registers: warps 0-3 hold K K^T, warps 4-7 hold Q K^T, 16 rows each
  const int mt = w & 3;
  float gram[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) gram[n][0] = gram[n][1] = gram[n][2] = gram[n][3] = 0.f;
  const int n_used = 2 * mt + 2;        // column tiles at or below the diagonal of row block mt; the rest is masked
  warp_gemm_nk_ldm<8, 16>(gram, (w < 4 ? Ks : Qs) + mt * 16 * kLdK, kLdK, Ks, kLdK, n_used);

  // ---- 3. per value head
  for (int vi = 0; vi < rep; ++vi) {
    const int h = kh * rep + vi;
    const size_t unit = (size_t)h * ws.chunks + c;
    const float* Gv = Gs + vi * 64; const float* bv = bs + vi * 64; const float* ev = es + vi * 64;
    __syncthreads();                    // previous head done with LT and the staging tile; qhat no longer needed
    {   // L (warps 0-3) and QKd (warps 4-7) straight from the Gram fragments
      float* qkd = ws.QKp + unit * 4096;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
          const int row = mt * 16 + g + 8 * hrow, col = n * 8 + 2 * tq;
          if (n >= n_used) {            // above the diagonal: nothing reads L there, QKd is zero
            if (w >= 4) *reinterpret_cast<float2*>(qkd + ((col >> 2) * 64 + row) * 4 + (col & 3)) = make_float2(0.f, 0.f);
            continue;
          }
          const float Gr = Gv[row];
          const float p0 = __expf(fminf(Gr - Gv[col], 0.f)), p1 = __expf(fminf(Gr - Gv[col + 1], 0.f));
          const float v0 = gram[n][2 * hrow], v1 = gram[n][2 * hrow + 1];
          if (w < 4) {
            const float b = bv[row];
            *reinterpret_cast<float2*>(LT + row * kLdM + col) = make_float2(col < row ? b * v0 * p0 : 0.f, col + 1 < row ? b * v1 * p1 : 0.f);
          } else {
            const int at = ((col >> 2) * 64 + row) * 4 + (col & 3);
            *reinterpret_cast<float2*>(qkd + at) = make_float2(col <= row ? tf32r(v0 * p0) : 0.f, col + 1 <= row ? tf32r(v1 * p1) : 0.f);
          }
        }
    }
    for (int i = t; i < 64 * 32; i += 256) {   // X = beta e^G K
      const int row = i >> 5, c4 = (i & 31) * 4;
      const float4 kv = *reinterpret_cast<const float4*>(Ks + row * kLdK + c4);
      const float e = ev[row];
      *reinterpret_cast<float4*>(Qs + row * kLdX + c4) = make_float4(tf32r(e * kv.x), tf32r(e * kv.y), tf32r(e * kv.z), tf32r(e * kv.w));
    }
    // raw v rows of value head h, 128 channels per round with bf16 inputs (already in flight), 64 with fp32 inputs
    constexpr int VCH = BF16 ? 128 : 64;
    if constexpr (BF16) cp_async_wait_all();
    else stage_raw<BF16, VCH>(P, C, r0, 2 * KW + h * 128, RB);
    __syncthreads();
    invert_unit_lower_64(LT, Ms);       // ends with a barrier; T stays fp32 and is rounded as the products load it
    // T is lower triangular: row block m needs k < 16 (m + 1).  A warp takes 32 columns of two row blocks, (3, 0) or
    // (2, 1), ten k steps either way.
    const int qn = w & 3, m_hi = w < 4 ? 3 : 2, m_lo = w < 4 ? 0 : 1;
    {   // W = T X
      float acc[2][4][4];
#pragma unroll
      for (int k = 0; k < 2; ++k)
#pragma unroll
        for (int n = 0; n < 4; ++n) acc[k][n][0] = acc[k][n][1] = acc[k][n][2] = acc[k][n][3] = 0.f;
      warp_gemm_tril_pair<4, true>(acc[0], acc[1], LT, kLdM, m_hi, m_lo, Qs + qn * 32, kLdX);
      float* dst = ws.WQ + unit * 16384;
#pragma unroll
      for (int k = 0; k < 2; ++k)
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const int col = qn * 32 + n * 8 + 2 * tq, r_lo = (k ? m_lo : m_hi) * 16 + g;
          *reinterpret_cast<float2*>(dst + ((col >> 2) * 128 + r_lo) * 4 + (col & 3)) = make_float2(tf32r(acc[k][n][0]), tf32r(acc[k][n][1]));
          *reinterpret_cast<float2*>(dst + ((col >> 2) * 128 + r_lo + 8) * 4 + (col & 3)) = make_float2(tf32r(acc[k][n][2]), tf32r(acc[k][n][3]));
        }
    }
    __syncthreads();                    // X = beta e^G K consumed
    for (int round = 0; round < 128 / VCH; ++round) {   // X = beta SiLU(conv(v)) from the staged raw rows
      if (round) {
        __syncthreads();
        stage_raw<BF16, VCH>(P, C, r0, 2 * KW + h * 128 + round * VCH, RB);
        __syncthreads();
      }
      constexpr int VP = VCH / 2, VSEG = 256 / VP, VR = 64 / VSEG;
      const int cp = t % VP, seg = t / VP, chl = 2 * cp, chg = 2 * KW + h * 128 + round * VCH + chl, rb = seg * VR;
      const float4 w0 = *reinterpret_cast<const float4*>(a.conv + (size_t)chg * 4);
      const float4 w1 = *reinterpret_cast<const float4*>(a.conv + (size_t)(chg + 1) * 4);
      float2 x0 = staged_pair<BF16>(RB, VCH, rb, chl), x1 = staged_pair<BF16>(RB, VCH, rb + 1, chl), x2 = staged_pair<BF16>(RB, VCH, rb + 2, chl);
#pragma unroll
      for (int i = 0; i < VR; ++i) {
        const float2 x3 = staged_pair<BF16>(RB, VCH, rb + 3 + i, chl);
        float c0 = w0.x * x0.x, c1 = w1.x * x0.y;
        c0 = fmaf(w0.y, x1.x, c0); c1 = fmaf(w1.y, x1.y, c1);
        c0 = fmaf(w0.z, x2.x, c0); c1 = fmaf(w1.z, x2.y, c1);
        c0 = fmaf(w0.w, x3.x, c0); c1 = fmaf(w1.w, x3.y, c1);
        const float b = rb + i < valid ? bv[rb + i] : 0.f;
        *reinterpret_cast<float2*>(Qs + (rb + i) * kLdX + round * VCH + chl) = make_float2(tf32r(b * siluf_(c0)), tf32r(b * siluf_(c1)));
        x0 = x1; x1 = x2; x2 = x3;
      }
    }
    __syncthreads();
    if constexpr (BF16) {   // staging tile consumed: start the next value head's rows
      if (vi + 1 < rep) stage_issue<true, 128>(P, C, r0, 2 * KW + (h + 1) * 128, RB);
    }
    {   // Ut = T X  (stored fp32: it is added, not multiplied, in the scan)
      float acc[2][4][4];
#pragma unroll
      for (int k = 0; k < 2; ++k)
#pragma unroll
        for (int n = 0; n < 4; ++n) acc[k][n][0] = acc[k][n][1] = acc[k][n][2] = acc[k][n][3] = 0.f;
      warp_gemm_tril_pair<4, true>(acc[0], acc[1], LT, kLdM, m_hi, m_lo, Qs + qn * 32, kLdX);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int mt2 = k ? m_lo : m_hi;
        // [token / 16][(token % 16) / 4][column][token % 4]: a scan thread owns a column and reads four tokens per
        // 128-bit load, a warp 512 contiguous bytes
        float* dst = ws.Ut + unit * 8192 + (size_t)mt2 * 2048;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const int col = qn * 32 + n * 8 + 2 * tq;
          float* d = dst + (g >> 2) * 512 + col * 4 + (g & 3);
          d[0] = acc[k][n][0]; d[4] = acc[k][n][1]; d[1024] = acc[k][n][2]; d[1028] = acc[k][n][3];
        }
      }
    }
  }
}

cr_status gdn_chunk_local_launch(const cr_geometry* g, const GdnPrefillParams& P, const ChunkWs& ws, bool bf16_in, cudaStream_t stream) {
  static PerDeviceOnce configured;
  if (cr_status st = once_per_device(configured, [] {
        CR_CUDA(cudaFuncSetAttribute(gdn_chunk_local_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLocalSmem));
        CR_CUDA(cudaFuncSetAttribute(gdn_chunk_local_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLocalSmem));
        return CR_OK;
      })) return st;
  const dim3 grid(ws.chunks, g->gdn_kheads);
  if (bf16_in) gdn_chunk_local_kernel<true><<<grid, 256, kLocalSmem, stream>>>(P, ws);
  else gdn_chunk_local_kernel<false><<<grid, 256, kLocalSmem, stream>>>(P, ws);
  CR_LAUNCH_CHECK("gdn_chunk_local_kernel");
  return CR_OK;
}

}  // namespace cr
