// Latent attention on the tensor cores (bf16 serving): every query head reads the SAME cache row per key -- the latent
// (key and value at once) followed by the rotated key part -- so the rows of a tile are (token, head) pairs and a key tile
// staged once in shared memory serves all heads.  Flash-attention form with mma.sync.m16n8k16 (bf16 operands, fp32 scores,
// softmax and accumulators): S = Q K^T over the whole cache row, O += P V over the latent columns of the same tile.
//
//   rows r = token * H + head, 16 per warp, WARPS warps per block; queries fp32 [T * H][W] (already in the cache's space:
//   hy_head_mm_t_kernel + hy_latent_prep_kernel), rounded to bf16 in shared memory
//   pool [n_pages * page_tokens][W] bf16, W = R + rot, W and R multiples of 16
//   grid (ceil(T * H / (16 * WARPS)), n_splits, ceil(R / DVC)): a block takes the tile's rows, one share of every
//   sequence's keys (n_splits equal shares, whole key tiles) and DVC value columns
//   n_splits == 1: out[t][h * R + c] = O / l;  else part[split][r][2 + R] = (m, l, O) and hy_latent_merge_kernel finishes.
// A tile's tokens may belong to several sequences (a batch of single tokens): the block walks them one after the other,
// rows of other sequences are masked for that walk.  Causal: row (t, h) sees keys at positions <= pos(t).
#pragma once
#include "xb_attn_mma.cuh"

#define HY_LAT_KEYS 32   // keys per shared-memory tile; two tiles are resident (the next one arrives by cp.async while this one is used)
#define HY_LAT_NEG -1.0e30f

// 16 bytes global -> shared without passing registers; bytes = 0 writes zeros instead (rows and columns outside the cache)
__device__ __forceinline__ void lat_cp16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lat_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void lat_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// LOADW >= WARPS warps per block: all of them stage queries and key tiles, the first WARPS own rows.
template <int WARPS, int DVC, int LOADW>
__global__ void __launch_bounds__(32 * LOADW) hy_latent_attn_mma_kernel(const float* __restrict__ qa, const bf16* __restrict__ pool, BatchMeta m,
                                                                        int T, int H, int W, int R, float scale_log2, int n_splits,
                                                                        float* __restrict__ part, float* __restrict__ out, long long ld_out) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char lsm[];
  constexpr int ROWS = 16 * WARPS, NT = 32 * LOADW, NDV = DVC / 8, NB = HY_LAT_KEYS / 8, KK = HY_LAT_KEYS / 16;
  const int Wp = (W + 15) & ~15, PITCH = Wp + 8;     // bf16 elements per shared row; the 16-byte pad keeps ldmatrix conflict-free
  bf16* Qs = reinterpret_cast<bf16*>(lsm);
  bf16* Kbuf = Qs + (size_t)ROWS * PITCH;     // two tiles of HY_LAT_KEYS rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const int NR = T * H;
  const int r0 = blockIdx.x * ROWS;
  const int split = blockIdx.y, c0 = blockIdx.z * DVC;
  const int ndv = (R - c0) / 8 < NDV ? (R - c0) / 8 : NDV;    // value column blocks of 8 that exist in this share
  // queries -> bf16 rows (zero beyond the batch and in the pad columns)
  for (int i = threadIdx.x; i < ROWS * (PITCH / 2); i += NT) {
    const int r = i / (PITCH / 2), c = (i - r * (PITCH / 2)) * 2;
    float2 v = make_float2(0.f, 0.f);
    if (r0 + r < NR && c < W) v = *reinterpret_cast<const float2*>(qa + (long long)(r0 + r) * W + c);
    *reinterpret_cast<uint32_t*>(Qs + (size_t)r * PITCH + c) = f2_to_bf2(v.x, v.y);
  }
  // this thread's two rows
  int rpos[2], rseq[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int r = r0 + warp * 16 + g + 8 * j;
    const int t = (r < NR && warp < WARPS) ? r / H : -1;
    rpos[j] = t >= 0 ? m.tok_pos[t] : -1;
    rseq[j] = t >= 0 ? m.tok_seq[t] : -1;
  }
  const int t_first = r0 / H, t_last = ((r0 + ROWS - 1 < NR ? r0 + ROWS - 1 : NR - 1)) / H;
  const int s_first = m.tok_seq[t_first], s_last = m.tok_seq[t_last];
  float mx[2] = {HY_LAT_NEG, HY_LAT_NEG}, ls[2] = {0.f, 0.f};
  float oacc[NDV][4];
#pragma unroll
  for (int n = 0; n < NDV; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
  // warp-level: does any of the warp's rows belong to the batch at all
  const int wr0 = r0 + warp * 16;
  for (int s = s_first; s <= s_last; ++s) {
    // newest position among the tile's tokens of sequence s (tokens of a sequence are contiguous and rising)
    int tl = t_last;
    while (tl > t_first && m.tok_seq[tl] != s) --tl;
    const int pmax = m.tok_pos[tl];
    const int* pages = m.page_table + (long long)m.seq_slot[s] * m.max_pages;
    // this block's share of keys [k_lo, k_hi): whole tiles
    const int tiles = (pmax + HY_LAT_KEYS) / HY_LAT_KEYS;
    const int per = (tiles + n_splits - 1) / n_splits;
    const int k_lo = split * per * HY_LAT_KEYS;
    int k_hi = (split + 1) * per * HY_LAT_KEYS;
    k_hi = k_hi < pmax + 1 ? k_hi : pmax + 1;
    // does this warp hold a row of s
    int wt0 = wr0 / H, wt1 = (wr0 + 15 < NR ? wr0 + 15 : NR - 1) / H;
    bool warp_active = false;
    if (wr0 < NR && warp < WARPS)
      for (int t = wt0; t <= wt1; ++t) warp_active = warp_active || m.tok_seq[t] == s;
    const int c8 = W >> 3;
    auto issue = [&](int kb, bf16* buf) {
      for (int i = threadIdx.x; i < HY_LAT_KEYS * (PITCH >> 3); i += NT) {
        const int k = i / (PITCH >> 3), c = i - k * (PITCH >> 3);
        const int kp = kb + k;
        const bool ok = kp < k_hi && c < c8;
        const bf16* src = pool;
        if (ok) src = pool + ((long long)pages[kp / m.page_tokens] * m.page_tokens + kp % m.page_tokens) * W + c * 8;
        lat_cp16(smem_u32(buf + (size_t)k * PITCH + c * 8), src, ok ? 16 : 0);
      }
      lat_cp_commit();
    };
    __syncthreads();       // nobody still reads a tile of the previous sequence; the queries are in place
    if (k_lo < k_hi) issue(k_lo, Kbuf);
    int cur = 0;
    for (int kb = k_lo; kb < k_hi; kb += HY_LAT_KEYS, cur ^= 1) {
      bf16* Ks = Kbuf + (size_t)cur * HY_LAT_KEYS * PITCH;
      if (kb + HY_LAT_KEYS < k_hi) {
        issue(kb + HY_LAT_KEYS, Kbuf + (size_t)(cur ^ 1) * HY_LAT_KEYS * PITCH);
        lat_cp_wait<1>();
      } else {
        lat_cp_wait<0>();
      }
      __syncthreads();     // this tile has arrived for every thread
      if (warp_active) {
      // ---- S = Q K^T, 16 rows x HY_LAT_KEYS keys per warp
      float sacc[NB][4];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
      const uint32_t qaddr = smem_u32(Qs + (size_t)(warp * 16 + (lane & 15)) * PITCH + (lane >> 4) * 8);
      const uint32_t kaddr = smem_u32(Ks + (size_t)((lane & 7) + ((lane >> 4) & 1) * 8) * PITCH + ((lane >> 3) & 1) * 8);
      for (int ks = 0; ks < Wp; ks += 16) {
        uint32_t a[4];
        ldsm_x4(qaddr + ks * 2, a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int nb = 0; nb < NB; nb += 2) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(kaddr + (uint32_t)(nb * 8 * PITCH + ks) * 2, b0, b1, b2, b3);
          mma_bf16_16816(sacc[nb], a, b0, b1);
          mma_bf16_16816(sacc[nb + 1], a, b2, b3);
        }
      }
      // ---- mask, online softmax (fp32, base 2)
      float tmax[2] = {HY_LAT_NEG, HY_LAT_NEG};
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = e >> 1, kp = kb + nb * 8 + 2 * q + (e & 1);
          const bool ok = rseq[j] == s && kp <= rpos[j];
          const float v = ok ? sacc[nb][e] * scale_log2 : HY_LAT_NEG;
          sacc[nb][e] = v;
          tmax[j] = fmaxf(tmax[j], v);
        }
      float corr[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 1));
        tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 2));
        const float nm = fmaxf(mx[j], tmax[j]);
        corr[j] = exp2f(mx[j] - nm);
        mx[j] = nm;
        ls[j] *= corr[j];
      }
      uint32_t pa[KK][4];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = e >> 1;
          p[e] = sacc[nb][e] > 0.5f * HY_LAT_NEG ? exp2f(sacc[nb][e] - mx[j]) : 0.f;
          ls[j] += p[e];
        }
        pa[nb >> 1][(nb & 1) * 2] = f2_to_bf2(p[0], p[1]);
        pa[nb >> 1][(nb & 1) * 2 + 1] = f2_to_bf2(p[2], p[3]);
      }
#pragma unroll
      for (int n = 0; n < NDV; ++n) {
        oacc[n][0] *= corr[0]; oacc[n][1] *= corr[0]; oacc[n][2] *= corr[1]; oacc[n][3] *= corr[1];
      }
      // ---- O += P V: V = the latent columns [c0, c0 + DVC) of the same tile
      const uint32_t vaddr = smem_u32(Ks + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + c0 + ((lane >> 4) & 1) * 8);
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
        for (int n = 0; n < NDV; n += 2) {
          if (n < ndv) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(vaddr + (uint32_t)(kk * 16 * PITCH + n * 8) * 2, b0, b1, b2, b3);
            mma_bf16_16816(oacc[n], pa[kk], b0, b1);
            mma_bf16_16816(oacc[n + 1], pa[kk], b2, b3);
          }
        }
      }
      }
      __syncthreads();     // every warp is done with this tile before the copy after next overwrites it
    }
  }
  // ---- results
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    ls[j] += __shfl_xor_sync(0xffffffffu, ls[j], 1);
    ls[j] += __shfl_xor_sync(0xffffffffu, ls[j], 2);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int r = r0 + warp * 16 + g + 8 * j;
    if (r >= NR || warp >= WARPS) continue;
    if (n_splits == 1) {
      const int t = r / H, h = r - t * H;
      const float inv = 1.0f / ls[j];
      float* dst = out + (long long)t * ld_out + (long long)h * R + c0;
#pragma unroll
      for (int n = 0; n < NDV; ++n)
        if (n < ndv) *reinterpret_cast<float2*>(dst + n * 8 + 2 * q) = make_float2(oacc[n][2 * j] * inv, oacc[n][2 * j + 1] * inv);
    } else {
      float* dst = part + ((long long)split * NR + r) * (R + 2);
      if (q == 0 && blockIdx.z == 0) { dst[0] = mx[j]; dst[1] = ls[j]; }
#pragma unroll
      for (int n = 0; n < NDV; ++n)
        if (n < ndv) *reinterpret_cast<float2*>(dst + 2 + c0 + n * 8 + 2 * q) = make_float2(oacc[n][2 * j], oacc[n][2 * j + 1]);
    }
  }
}

// out[t][h * R + c] = sum_s O_s[c] 2^(m_s - M) / sum_s l_s 2^(m_s - M), M = max_s m_s.  grid (T * H), 128 threads.
__global__ void __launch_bounds__(128) hy_latent_merge_kernel(const float* __restrict__ part, int n_splits, int NR, int H, int R,
                                                              float* __restrict__ out, long long ld_out) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int t = r / H, h = r - t * H;
  float M = HY_LAT_NEG;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part[((long long)s * NR + r) * (R + 2)]);
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float* p = part + ((long long)s * NR + r) * (R + 2);
    L += p[1] * exp2f(p[0] - M);
  }
  const float inv = 1.0f / L;
  for (int c = threadIdx.x; c < R; c += 128) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float* p = part + ((long long)s * NR + r) * (R + 2);
      acc = fmaf(p[2 + c], exp2f(p[0] - M), acc);
    }
    out[(long long)t * ld_out + (long long)h * R + c] = acc * inv;
  }
}
