// Tensor-core version of the pooled-window attention (see pooled_window_attention.cu for the mechanism and the cache
// layout), bf16 cache, for prompt portions and for decoded tokens alike.
//
// CTA = one tile of up to 16 consecutive tokens of a sequence with ALL heads (the mixing of softmax weights across
// heads needs every head's weight for a key), 4 to 16 warps.  Per tile of 32 keys (pooled rows first, then the window's
// tokens; rows come straight from the paged cache by 16-byte cp.async, into two stages where shared memory allows, so
// that the next tile's copies fly during this tile's products):
//   scores   S_g = Q_g K^T for every head g, heads dealt out to the warps: mma.sync m16n8k16, fp32 accumulation.  The
//            fp32 queries (already scaled by scale * temp[g]) are held as a bf16 pair hi + lo while that fits in shared
//            memory, so the products are exact to ~2^-17; beyond that size as one bf16.
//   pass 0   running maximum and sum of every (head, token) row, in shared memory.
//   pass 1   normalised weights exp(s - m) / l of all heads to shared memory in fp32; each warp then owns one (head,
//            block of output columns): it forms its head's MIXED weights sum_g talk[h][g] w_g directly in the A-fragment
//            layout (fp32), splits them into a bf16 pair and multiplies both halves with the value tile (ldmatrix with
//            transposition), accumulating the output in registers.
// Scores, softmax, mixing and all sums are fp32.  Rows of a tile beyond its tokens read a zero query row.
// Reference: none (the reference has no attention code; reference llmctl/serve/server.py:199-204 calls HF).
#include "../common/dtype.cuh"
#include "../common/mma_sync.cuh"
#include "pooled_window.cuh"

namespace llmctl {

constexpr int kMTK = 32;      // keys per tile
constexpr int kPld = 40;      // row pitch of the weight tiles (floats): conflict-free 8-byte fragment reads

struct PwaMmaParams {
  const float* q;
  const __nv_bfloat16* cache;
  const int* block_tables;
  int max_blocks;
  const int* tiles;
  const int* positions;
  const float* temp;
  const float* talk;
  float scale;
  int H, G, d, e, S, P, bs, PS;
  int qrows;        // query rows held in shared memory (tile tokens + one zero row)
  int qlo;          // 1: queries as hi + lo
  int stages;       // 2: key/value tiles double-buffered, the next tile's copies fly during this tile's products
  int nwarps;
  int chunks;       // blocks of NT * 8 output columns per head
  __nv_bfloat16* out;
  // keys split over `splits` CTAs per tile (few tiles, long contexts: decoding).  mode 0: one CTA does both passes;
  // mode 1: pass 0 over the CTA's slice, (max, sum) of every row to part_ml; mode 2: pass 1 over the slice with the
  // slices' (max, sum) combined, fp32 partial outputs to part_o [splits, tokens, H*e] (they simply add up, since the
  // weights are normalised with the global sum)
  int splits, mode, tokens;
  float* part_ml;   // [tiles, splits, H*16, 2]
  float* part_o;
};

__device__ __forceinline__ uint32_t pack_bf16(__nv_bfloat16 a, __nv_bfloat16 b) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(a)) | (static_cast<uint32_t>(__bfloat16_as_ushort(b)) << 16);
}

// ldmatrix on a shared-memory byte address (the per-lane row addresses are formed once, outside the loops).
__device__ __forceinline__ void ldsm_x4(uint32_t (&a)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&b)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(b[0]), "=r"(b[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&b)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(b[0]), "=r"(b[1]) : "r"(addr));
}

template <int NT>
__global__ void __launch_bounds__(512)
pooled_window_attention_mma_kernel(const PwaMmaParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, G = p.G, d = p.d, e = p.e, S = p.S, P = p.P, bs = p.bs, PS = p.PS;
  const int rep = H / G, Wc = G * (d + e);
  const int tile = blockIdx.x / p.splits, split = blockIdx.x % p.splits;
  const int t0 = p.tiles[tile * 4], nq = p.tiles[tile * 4 + 1];
  if (nq <= 0) return;
  const int* table = p.block_tables + static_cast<long long>(p.tiles[tile * 4 + 2]) * p.max_blocks;
  const int p_first = p.positions[t0], p_last = p_first + nq - 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = p.nwarps * 32;
  const int row = lane >> 2, tq = lane & 3;

  const int ldq = H * d + 8, ldk = G * d + 8, ldv = G * e + 8;
  __nv_bfloat16* Qhi = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [qrows][ldq]
  __nv_bfloat16* Qlo = Qhi + (p.qlo ? p.qrows * ldq : 0);                           // [qrows][ldq] when qlo
  __nv_bfloat16* Ks = Qlo + p.qrows * ldq;                                          // [stages][kMTK][ldk]
  __nv_bfloat16* Vs = Ks + p.stages * kMTK * ldk;                                   // [stages][kMTK][ldv]
  float* Pw = reinterpret_cast<float*>(Vs + p.stages * kMTK * ldv);                 // [H][16][kPld]
  float* sM = Pw + H * 16 * kPld;                                                   // [H][16]
  float* sL = sM + H * 16;                                                          // [H][16]
  float* sTalk = sL + H * 16;                                                       // [H][H]
  int* klo = reinterpret_cast<int*>(sTalk + H * H);                                 // [stages][kMTK]
  int* khi = klo + p.stages * kMTK;
  int* krow = khi + p.stages * kMTK;

  const int zrow = p.qrows - 1;
  // scores are kept in units of ln 2 (log2(e) folded into the query scaling), so that every exponential is one exp2f
  for (int r = warp; r < p.qrows; r += p.nwarps) {              // a warp per query row, four numbers per lane and step
    const float4* src = reinterpret_cast<const float4*>(p.q + static_cast<long long>(t0 + (r < nq ? r : 0)) * H * d);
#pragma unroll 4
    for (int c4 = lane; c4 < (H * d) >> 2; c4 += 32) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < nq) {
        v = src[c4];
        const float f = p.scale * (p.temp ? p.temp[(c4 << 2) / d] : 1.f) * 1.4426950408889634f;
        v.x *= f, v.y *= f, v.z *= f, v.w *= f;
      }
      const __nv_bfloat16 h0 = __float2bfloat16(v.x), h1 = __float2bfloat16(v.y), h2 = __float2bfloat16(v.z), h3 = __float2bfloat16(v.w);
      *reinterpret_cast<uint2*>(Qhi + r * ldq + (c4 << 2)) = make_uint2(pack_bf16(h0, h1), pack_bf16(h2, h3));
      if (p.qlo)
        *reinterpret_cast<uint2*>(Qlo + r * ldq + (c4 << 2)) =
            make_uint2(pack_bf16(__float2bfloat16(v.x - __bfloat162float(h0)), __float2bfloat16(v.y - __bfloat162float(h1))),
                       pack_bf16(__float2bfloat16(v.z - __bfloat162float(h2)), __float2bfloat16(v.w - __bfloat162float(h3))));
    }
  }
  for (int i = tid; i < H * 16; i += nthreads) {
    sM[i] = -INFINITY;
    sL[i] = 0.f;
  }
  if (p.talk)
    for (int i = tid; i < H * H; i += nthreads) sTalk[i] = p.talk[i];

  const int nb = (S > 0 && p_last - S + 1 >= P) ? (p_last - S + 1) / P : 0;
  const int j0 = (S > 0 && p_first - S + 1 > 0) ? p_first - S + 1 : 0;
  const int NU = nb + (p_last - j0 + 1);

  constexpr int kUnits = 16 / NT;       // (head, column block) units per warp: 16 n-tiles of accumulators in all
  float oacc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) oacc[i][j] = 0.f;

  // per-lane ldmatrix addresses (bytes in shared memory): query rows beyond the tile alias the zero row
  const uint32_t q_lane = ((((lane & 15) < nq ? (lane & 15) : zrow) * ldq + ((lane >> 4) << 3)) << 1);
  const uint32_t qhi_addr = static_cast<uint32_t>(__cvta_generic_to_shared(Qhi)) + q_lane;
  const uint32_t qlo_addr = static_cast<uint32_t>(__cvta_generic_to_shared(Qlo)) + q_lane;
  const uint32_t k_addr = static_cast<uint32_t>(__cvta_generic_to_shared(Ks)) + ((((lane & 7) * ldk) + (((lane >> 3) & 1) << 3)) << 1);
  const uint32_t v_addr = static_cast<uint32_t>(__cvta_generic_to_shared(Vs)) + (((lane & 15) * ldv) << 1);
  const int kchunks = (G * d) >> 3, vchunks = (G * e) >> 3;      // 16-byte pieces per key / value row
  const int per = ((NU + kMTK - 1) / kMTK + p.splits - 1) / p.splits * kMTK;      // keys per slice, whole tiles
  const int u_begin = split * per, u_end = min(NU, u_begin + per);
  if (p.mode == 2) {
    __syncthreads();
    for (int i = tid; i < H * 16; i += nthreads) {
      const float* ml = p.part_ml + (static_cast<long long>(tile) * p.splits * H * 16 + i) * 2;
      float m = -INFINITY, l = 0.f;
      for (int s2 = 0; s2 < p.splits; ++s2) m = fmaxf(m, ml[static_cast<long long>(s2) * H * 16 * 2]);
      if (m > -INFINITY)
        for (int s2 = 0; s2 < p.splits; ++s2) l += ml[static_cast<long long>(s2) * H * 16 * 2 + 1] * exp2f(ml[static_cast<long long>(s2) * H * 16 * 2] - m);
      sM[i] = m;
      sL[i] = l > 0.f ? 1.f / l : 0.f;
    }
  }
  for (int pass = (p.mode == 2 ? 1 : 0); pass < (p.mode == 1 ? 1 : 2); ++pass) {
    // Tile `it` lives in stage it % stages.  fetch(): visibility and cache rows of the tile's keys, then its copies (one
    // cp.async group per tile); returns whether all 16 tokens see the whole tile (no mask to apply then).
    auto fetch = [&](int it, int st) -> bool {
      const int u0 = u_begin + it * kMTK;
      const int nk = min(kMTK, NU - u0);
      int all_seen = 1;
      if (tid < kMTK) {
        const WindowKey k = window_key(table, u0 + tid, nb, j0, NU, S, P, bs, PS);
        klo[st * kMTK + tid] = k.lo;
        khi[st * kMTK + tid] = k.hi;
        krow[st * kMTK + tid] = k.row;
        all_seen = k.lo <= p_first && k.hi >= p_last;
      }
      const bool whole = __syncthreads_and(all_seen) && nq == 16;
      __nv_bfloat16* kd = Ks + st * kMTK * ldk;
      __nv_bfloat16* vd = Vs + st * kMTK * ldv;
      for (int k = warp; k < kMTK; k += p.nwarps) {       // a warp per cache row, a lane per 16-byte piece
        const __nv_bfloat16* src = p.cache + static_cast<long long>(krow[st * kMTK + k]) * Wc;
        for (int c = lane; c < kchunks; c += 32) {
          if (k < nk) cp_async_16(kd + k * ldk + c * 8, src + c * 8);
          else *reinterpret_cast<uint4*>(kd + k * ldk + c * 8) = make_uint4(0, 0, 0, 0);
        }
        if (pass == 1)
          for (int c = lane; c < vchunks; c += 32) {
            if (k < nk) cp_async_16(vd + k * ldv + c * 8, src + G * d + c * 8);
            else *reinterpret_cast<uint4*>(vd + k * ldv + c * 8) = make_uint4(0, 0, 0, 0);
          }
      }
      cp_async_commit();
      return whole;
    };
    const int n_tiles = u_end > u_begin ? (u_end - u_begin + kMTK - 1) / kMTK : 0;
    __syncthreads();                                    // the previous pass is done with every stage
    bool unmasked_next = n_tiles > 0 ? fetch(0, 0) : false;
    for (int it = 0; it < n_tiles; ++it) {
      const int st = p.stages == 2 ? (it & 1) : 0;
      const bool unmasked = unmasked_next;
      if (p.stages == 2 && it + 1 < n_tiles) {
        unmasked_next = fetch(it + 1, st ^ 1);          // stage st ^ 1 was released by the barrier that ended tile it - 1
        cp_async_wait_prior();                          // tile it has landed; tile it + 1 is in flight
      } else {
        cp_async_wait_all();
      }
      __syncthreads();
      const int* tlo = klo + st * kMTK;
      const int* thi = khi + st * kMTK;
      const uint32_t k_stage = k_addr + ((st * kMTK * ldk) << 1), v_stage = v_addr + ((st * kMTK * ldv) << 1);

      // ---- scores of the heads this warp is dealt ----
      for (int g = warp; g < H; g += p.nwarps) {
        const int c = g / rep;
        float sacc[kMTK / 8][4];
#pragma unroll
        for (int nt = 0; nt < kMTK / 8; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) sacc[nt][j] = 0.f;
        const uint32_t qa = qhi_addr + ((g * d) << 1), qb = qlo_addr + ((g * d) << 1), ka = k_stage + ((c * d) << 1);
        const uint32_t kstep = (8 * ldk) << 1;                      // bytes between n-tiles of 8 keys
#pragma unroll 2
        for (int ks = 0; ks < d; ks += 16) {
          uint32_t ahi[4], alo[4];
          ldsm_x4(ahi, qa + (ks << 1));
          if (p.qlo) ldsm_x4(alo, qb + (ks << 1));
#pragma unroll
          for (int nt = 0; nt < kMTK / 8; ++nt) {
            uint32_t b[2];
            ldsm_x2(b, ka + (ks << 1) + nt * kstep);
            mma_bf16_16816(sacc[nt], ahi, b);
            if (p.qlo) mma_bf16_16816(sacc[nt], alo, b);
          }
        }
        // element j of n-tile nt: row = row + 8 * (j / 2), key = nt * 8 + 2 * tq + (j & 1)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < kMTK / 8; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (!unmasked) {
              const int r = row + 8 * (j >> 1), k = nt * 8 + 2 * tq + (j & 1);
              const int pi = p_first + r;
              const bool seen = r < nq && pi >= tlo[k] && pi <= thi[k];
              sacc[nt][j] = seen ? sacc[nt][j] : -INFINITY;
            }
            mx[j >> 1] = fmaxf(mx[j >> 1], sacc[nt][j]);
          }
        if (pass == 0) {
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            float tm = mx[h2];
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
            const int r = row + 8 * h2;
            const float m_old = sM[g * 16 + r], l_old = sL[g * 16 + r];
            const float mn = fmaxf(m_old, tm);
            float add = 0.f;
            if (mn > -INFINITY) {
#pragma unroll
              for (int nt = 0; nt < kMTK / 8; ++nt) add += exp2f(sacc[nt][2 * h2] - mn) + exp2f(sacc[nt][2 * h2 + 1] - mn);
            }
            add += __shfl_xor_sync(0xffffffffu, add, 1);
            add += __shfl_xor_sync(0xffffffffu, add, 2);
            __syncwarp();
            if (tq == 0 && mn > -INFINITY) {
              sM[g * 16 + r] = mn;
              sL[g * 16 + r] = l_old * exp2f(m_old - mn) + add;       // 2^(-inf) = 0 at the first tile that shows a key
            }
          }
        } else {
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            const int r = row + 8 * h2;
            const float m = sM[g * 16 + r], il = sL[g * 16 + r];
#pragma unroll
            for (int nt = 0; nt < kMTK / 8; ++nt) {
              float2 w;
              w.x = sacc[nt][2 * h2] > -INFINITY ? exp2f(sacc[nt][2 * h2] - m) * il : 0.f;
              w.y = sacc[nt][2 * h2 + 1] > -INFINITY ? exp2f(sacc[nt][2 * h2 + 1] - m) * il : 0.f;
              *reinterpret_cast<float2*>(Pw + (g * 16 + r) * kPld + nt * 8 + 2 * tq) = w;
            }
          }
        }
      }
      if (pass == 0) {
        __syncthreads();                                  // the stage is free again
        if (p.stages == 1 && it + 1 < n_tiles) unmasked_next = fetch(it + 1, 0);
        continue;
      }
      __syncthreads();
      // ---- mixed weights x values, one (head, block of NT * 8 output columns) per warp at a time ----
#pragma unroll
      for (int iu = 0; iu < kUnits; ++iu) {
        const int unit = warp + iu * p.nwarps;
        if (unit >= H * p.chunks) break;
        const int h = unit / p.chunks, n_first = (unit % p.chunks) * NT;
        const int c = h / rep;
#pragma unroll
        for (int ks = 0; ks < kMTK; ks += 16) {
          float a[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] = 0.f;
          const float* base = Pw + row * kPld + ks + 2 * tq;
          if (p.talk) {
#pragma unroll 4
            for (int g = 0; g < H; ++g) {
              const float tg = sTalk[h * H + g];
              const float* pg = base + g * 16 * kPld;
              const float2 x0 = *reinterpret_cast<const float2*>(pg), x1 = *reinterpret_cast<const float2*>(pg + 8 * kPld);
              const float2 x2 = *reinterpret_cast<const float2*>(pg + 8), x3 = *reinterpret_cast<const float2*>(pg + 8 * kPld + 8);
              a[0] = fmaf(tg, x0.x, a[0]);
              a[1] = fmaf(tg, x0.y, a[1]);
              a[2] = fmaf(tg, x1.x, a[2]);
              a[3] = fmaf(tg, x1.y, a[3]);
              a[4] = fmaf(tg, x2.x, a[4]);
              a[5] = fmaf(tg, x2.y, a[5]);
              a[6] = fmaf(tg, x3.x, a[6]);
              a[7] = fmaf(tg, x3.y, a[7]);
            }
          } else {
            const float* pg = base + h * 16 * kPld;
            const float2 x0 = *reinterpret_cast<const float2*>(pg), x1 = *reinterpret_cast<const float2*>(pg + 8 * kPld);
            const float2 x2 = *reinterpret_cast<const float2*>(pg + 8), x3 = *reinterpret_cast<const float2*>(pg + 8 * kPld + 8);
            a[0] = x0.x, a[1] = x0.y, a[2] = x1.x, a[3] = x1.y, a[4] = x2.x, a[5] = x2.y, a[6] = x3.x, a[7] = x3.y;
          }
          uint32_t ahi[4], alo[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __nv_bfloat16 h0 = __float2bfloat16(a[2 * j]), h1 = __float2bfloat16(a[2 * j + 1]);
            ahi[j] = pack_bf16(h0, h1);
            alo[j] = pack_bf16(__float2bfloat16(a[2 * j] - __bfloat162float(h0)), __float2bfloat16(a[2 * j + 1] - __bfloat162float(h1)));
          }
          const uint32_t va = v_stage + ((ks * ldv + c * e + n_first * 8) << 1);
          const int n_live = min(NT, (e >> 3) - n_first);          // n-tiles of this unit that exist
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            if (nt >= n_live) break;
            uint32_t b[2];
            ldsm_x2_trans(b, va + nt * 16);
            mma_bf16_16816(oacc[iu * NT + nt], ahi, b);
            mma_bf16_16816(oacc[iu * NT + nt], alo, b);
          }
        }
      }
      __syncthreads();                                    // the stage and the weight tile are free again
      if (p.stages == 1 && it + 1 < n_tiles) unmasked_next = fetch(it + 1, 0);
    }
    if (pass == 0) {
      __syncthreads();
      if (p.mode == 1) {
        float* ml = p.part_ml + (static_cast<long long>(tile) * p.splits + split) * H * 16 * 2;
        for (int r = tid; r < H * 16; r += nthreads) {
          ml[2 * r] = sM[r];
          ml[2 * r + 1] = sL[r];
        }
        return;
      }
      for (int r = tid; r < H * 16; r += nthreads) sL[r] = sL[r] > 0.f ? 1.f / sL[r] : 0.f;     // 1 / sum from here on
    }
  }
#pragma unroll
  for (int iu = 0; iu < kUnits; ++iu) {
    const int unit = warp + iu * p.nwarps;
    if (unit >= H * p.chunks) break;
    const int h = unit / p.chunks, n_first = (unit % p.chunks) * NT;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if ((n_first + nt) * 8 >= e) break;
      const int col = h * e + (n_first + nt) * 8 + 2 * tq;
      const float* o = oacc[iu * NT + nt];
      if (p.mode == 2) {
        float* po = p.part_o + static_cast<long long>(split) * p.tokens * H * e;
        if (row < nq) *reinterpret_cast<float2*>(po + static_cast<long long>(t0 + row) * H * e + col) = make_float2(o[0], o[1]);
        if (row + 8 < nq) *reinterpret_cast<float2*>(po + static_cast<long long>(t0 + row + 8) * H * e + col) = make_float2(o[2], o[3]);
        continue;
      }
      if (row < nq)
        *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t0 + row) * H * e + col) =
            pack_bf16(__float2bfloat16(o[0]), __float2bfloat16(o[1]));
      if (row + 8 < nq)
        *reinterpret_cast<uint32_t*>(p.out + static_cast<long long>(t0 + row + 8) * H * e + col) =
            pack_bf16(__float2bfloat16(o[2]), __float2bfloat16(o[3]));
    }
  }
}

__global__ void __launch_bounds__(256)
pwa_sum_partials_kernel(const float* __restrict__ part, int splits, long long n, __nv_bfloat16* __restrict__ out) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += part[s * n + i];
  out[i] = __float2bfloat16(v);
}

static size_t pwa_mma_smem(int H, int G, int d, int e, int qrows, int qlo, int stages) {
  size_t b = static_cast<size_t>(qrows) * (H * d + 8) * 2 * (qlo ? 2 : 1) + static_cast<size_t>(stages) * kMTK * (G * d + 8 + G * e + 8) * 2;
  b += (static_cast<size_t>(H) * 16 * kPld + 2ull * H * 16 + static_cast<size_t>(H) * H) * 4 + 3ull * stages * kMTK * 4;
  return b;
}

// Output columns per unit (8 * NT, NT in {4, 8, 16}), warps per CTA and units per head for these sizes: a warp holds 16
// n-tiles of accumulators, i.e. up to 16 / NT units.  Returns 0 when the sizes do not fit this kernel.
static int pwa_mma_plan(int H, int G, int d, int e, int tile_tokens, int* nt_out, int* nwarps, int* chunks, int* qrows, int* qlo,
                        int* stages) {
  if (H % G || d % 16 || e % 8 || (G * d) % 8 || (G * (d + e)) % 8 || tile_tokens > 16) return 0;
  // A unit mixes its head's weights itself, so fewer, wider units per head mean less repeated mixing: the widest unit
  // that still leaves 8 units to spread over the warps; with few heads of few columns, the narrowest.
  int nt = 0, ch = 0;
  for (int cand : {16, 8, 4}) {
    const int c = (e / 8 + cand - 1) / cand;
    if (H * c <= 16 * (16 / cand) && (H * c >= 8 || cand == 4)) {
      nt = cand;
      ch = c;
      break;
    }
  }
  if (!nt) return 0;
  int w = 4;
  while (w < H * ch && w < 16) w <<= 1;
  *nt_out = nt;
  *nwarps = w;
  *chunks = ch;
  *qrows = tile_tokens + 1;
  // shared memory goes to the exact queries first, then to the second key/value stage, unless that stage would cost a
  // resident CTA (two CTAs that overlap each other's copies beat one CTA that overlaps its own)
  *qlo = pwa_mma_smem(H, G, d, e, *qrows, 1, 1) <= 200 * 1024;
  auto resident = [&](int stg) {
    const int by_smem = static_cast<int>((227 * 1024) / (pwa_mma_smem(H, G, d, e, *qrows, *qlo, stg) + 1024));
    const int by_regs = 65536 / (w * 32 * 128);
    return by_smem < by_regs ? by_smem : by_regs;
  };
  *stages = (pwa_mma_smem(H, G, d, e, *qrows, *qlo, 2) <= 200 * 1024 && resident(2) >= resident(1)) ? 2 : 1;
  return pwa_mma_smem(H, G, d, e, *qrows, *qlo, *stages) <= 200 * 1024;
}

}  // namespace llmctl

using namespace llmctl;

// 1 if llmctl_pooled_window_attention_mma takes these sizes (bf16 only).
LLMCTL_API int llmctl_pooled_window_attention_mma_ok(int H, int G, int d, int e, int tile_tokens) {
  int nt, w, ch, qr, ql, stg;
  return pwa_mma_plan(H, G, d, e, tile_tokens, &nt, &w, &ch, &qr, &ql, &stg);
}

// Same arguments as llmctl_pooled_window_attention; cache and out are bf16.  splits > 1 cuts every tile's keys into
// that many slices with a CTA each (three launches: row statistics, weighted values, sum of the slices) and needs
// part_ml: fp32 [ntiles * splits * H * 16 * 2] and part_o: fp32 [splits * tokens * H * e].
LLMCTL_API int llmctl_pooled_window_attention_mma(const float* q, const void* cache, const int* block_tables, int max_blocks,
                                                  const int* tiles, int ntiles, int tile_tokens, const int* positions,
                                                  const float* temp, const float* talk, float scale, int H, int G, int d, int e,
                                                  int S, int P, int bs, int PS, void* out, int splits, int tokens, float* part_ml,
                                                  float* part_o, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && G > 0 && d > 0 && e > 0 && S >= 0 && (S == 0 || P > 0) && bs > 0 && tile_tokens > 0);
  if (ntiles == 0) return 0;
  int nt, w, ch, qr, ql, stg;
  LLMCTL_REQUIRE(pwa_mma_plan(H, G, d, e, tile_tokens, &nt, &w, &ch, &qr, &ql, &stg));
  PwaMmaParams p{q, (const __nv_bfloat16*)cache, block_tables, max_blocks, tiles, positions, temp, talk, scale, H, G, d, e, S, P, bs, PS,
                 qr, ql, stg, w, ch, (__nv_bfloat16*)out, splits > 1 ? splits : 1, 0, tokens, part_ml, part_o};
  LLMCTL_REQUIRE(splits <= 1 || (part_ml != nullptr && part_o != nullptr && tokens > 0));
  const size_t smem = pwa_mma_smem(H, G, d, e, qr, ql, stg);
  cudaStream_t s = (cudaStream_t)stream;
#define LLMCTL_PWA_LAUNCH(NT)                                                                                              \
  do {                                                                                                                     \
    auto kern = pooled_window_attention_mma_kernel<NT>;                                                                    \
    LLMCTL_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));         \
    if (p.splits == 1) {                                                                                                   \
      kern<<<ntiles, w * 32, smem, s>>>(p);                                                                                \
    } else {                                                                                                               \
      p.mode = 1;                                                                                                          \
      kern<<<ntiles * p.splits, w * 32, smem, s>>>(p);                                                                     \
      p.mode = 2;                                                                                                          \
      kern<<<ntiles * p.splits, w * 32, smem, s>>>(p);                                                                     \
      const long long n = static_cast<long long>(tokens) * H * e;                                                          \
      pwa_sum_partials_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, s>>>(part_o, p.splits, n, (__nv_bfloat16*)out); \
    }                                                                                                                      \
  } while (0)
  if (nt == 4) LLMCTL_PWA_LAUNCH(4);
  else if (nt == 8) LLMCTL_PWA_LAUNCH(8);
  else LLMCTL_PWA_LAUNCH(16);
#undef LLMCTL_PWA_LAUNCH
  LLMCTL_RETURN_LAST();
}
