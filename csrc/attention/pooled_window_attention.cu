// Sliding-window attention with pooled far context over a paged cache, for ragged batches (portions of prompts next
// to single decoded tokens), bf16 or fp32.
//
// A query at position i sees the tokens j with 0 <= i - j < S and, beside them, ONE key and value per block of P
// tokens that lies wholly before its window (block b = positions bP .. bP+P-1, seen once bP+P-1 <= i - S): the mean of
// the block's cached keys and the mean of its cached values.  Tokens and blocks share one softmax.  H query heads use
// G key/value heads (head h reads head h / (H/G)); keys have d numbers per head, values e.
//
// Cache of a layer: [pages, bs + PS, G*(d+e)].  Rows 0..bs-1 of a page are its tokens ([keys of all heads | values of
// all heads]); rows bs.. are the pooled rows of the blocks whose first token lies in the page (PS = ceil(bs / P) of
// them at most), so pooled rows are owned, freed and reused with the page.
//
//   llmctl_window_qkv_write : per token, from the packed projection [q | k | v]: + bias, RMS norm over the whole q
//       and the whole k projection (per-coordinate weights), rotation of the first `rot` numbers of every head as
//       interleaved pairs at the token's position, value mixing v <- (1-lam) v + lam v_first with the values an
//       earlier layer computed for the same token; q leaves in fp32, k and v go to the token's cache row.
//   llmctl_window_pool_update : for every token of the step that completes a block, the block's pooled row.
//   llmctl_pooled_window_attention : scores * scale * temp[h] in fp32, softmax over the visible tokens and blocks,
//       optional mixing of the NORMALISED weights across heads (w'_h = sum_g talk[h,g] w_g), then w' V with the
//       values of h's own key/value head.  Two passes over the keys: the first finds each row's maximum and sum, the
//       second forms the normalised weights of ALL heads for a key tile, mixes them and accumulates.  A CTA owns TQ
//       consecutive tokens of one sequence with all their heads (the mixing needs every head's weight for a key).
//
// Everything but the cached keys/values and the output is fp32 (FMA): scores, softmax, mixed weights, accumulators.
// Reference: none (the reference has no attention code; reference llmctl/serve/server.py:199-204 calls HF).
#include <limits.h>

#include "../common/dtype.cuh"
#include "../rope/rope_interleaved.cuh"
#include "pooled_window.cuh"

namespace llmctl {

// ---------------------------------------------------------------------------------------------------------------
// projection post-processing + cache append: one CTA per token
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
window_qkv_write_kernel(const T* __restrict__ qkv, long long ld, const T* __restrict__ bias, const float* __restrict__ qn_w,
                        const float* __restrict__ kn_w, int H, int G, int d, int e, int rot, const float* __restrict__ freq,
                        float mult, float eps, const int* __restrict__ positions, const long long* __restrict__ slots,
                        float* __restrict__ q_out, T* __restrict__ cache, int bs, int PS, T* __restrict__ v_first, int v_mode,
                        const float* __restrict__ lam) {
  extern __shared__ float buf[];      // [H*d + G*d]
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int Nq = H * d, Nk = G * d, Nv = G * e, Wc = Nk + Nv;
  const T* row = qkv + t * ld;
  float* sq = buf;
  float* sk = buf + Nq;
  float ssq = 0.f, ssk = 0.f;
  for (int c = threadIdx.x; c < Nq + Nk; c += blockDim.x) {
    float v = to_f32(row[c]);
    if (bias) v += to_f32(bias[c]);
    buf[c] = v;
    if (c < Nq) ssq += v * v;
    else ssk += v * v;
  }
  ssq = block_sum(ssq, red);
  ssk = block_sum(ssk, red);
  const float rq = qn_w ? 1.f / sqrtf(ssq / static_cast<float>(Nq) + eps) : 1.f;
  const float rk = kn_w ? 1.f / sqrtf(ssk / static_cast<float>(Nk) + eps) : 1.f;
  for (int c = threadIdx.x; c < Nq + Nk; c += blockDim.x) {
    if (c < Nq) sq[c] = sq[c] * rq * (qn_w ? qn_w[c] : 1.f);
    else sk[c - Nq] = sk[c - Nq] * rk * (kn_w ? kn_w[c - Nq] : 1.f);
  }
  __syncthreads();
  const int pos = positions[t];
  const long long slot = slots[t];
  T* crow = slot >= 0 ? cache + ((slot / bs) * (bs + PS) + slot % bs) * Wc : nullptr;
  for (int c = threadIdx.x; c < Nq + Nk; c += blockDim.x) {
    const bool isq = c < Nq;
    const int cc = isq ? c : c - Nq;
    const float* src = isq ? sq : sk;
    const int dd = cc % d, base = cc - dd;
    float v = src[cc];
    if (dd < rot) v = rope_interleaved_coord([&](int k) { return src[base + k]; }, dd, pos, freq, mult);
    if (isq) q_out[t * Nq + cc] = v;
    else if (crow) crow[cc] = from_f32<T>(v);
  }
  const float l = (v_mode == 2) ? lam[0] : 0.f;
  for (int c = threadIdx.x; c < Nv; c += blockDim.x) {
    float v = to_f32(row[Nq + Nk + c]);
    if (bias) v += to_f32(bias[Nq + Nk + c]);
    const T vt = from_f32<T>(v);               // the projection's output in the activation type
    if (v_mode == 1) v_first[t * Nv + c] = vt;
    v = to_f32(vt);
    if (v_mode == 2) v = (1.f - l) * v + l * to_f32(v_first[t * Nv + c]);
    if (crow) crow[Nk + c] = from_f32<T>(v);
  }
}

// one CTA per token; only the tokens that end a block do anything
template <typename T>
__global__ void __launch_bounds__(128)
window_pool_update_kernel(T* __restrict__ cache, const int* __restrict__ positions, const long long* __restrict__ slots,
                          const int* __restrict__ seq_rows, const int* __restrict__ block_tables, int max_blocks, int bs, int PS,
                          int P, int Wc) {
  const int t = blockIdx.x;
  const int p = positions[t];
  if (slots[t] < 0 || (p + 1) % P != 0) return;
  const int b = p / P;
  const int* table = block_tables + static_cast<long long>(seq_rows[t]) * max_blocks;
  T* dst = cache + pooled_row(table, b, P, bs, PS) * Wc;
  for (int c = threadIdx.x; c < Wc; c += blockDim.x) {
    float s = 0.f;
    for (int j = b * P; j <= p; ++j) s += to_f32(cache[token_row(table, j, bs, PS) * Wc + c]);
    dst[c] = from_f32<T>(s / static_cast<float>(P));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------------------------
constexpr int kTK = 32;           // keys per tile
constexpr int kAcc = 32;          // output accumulators per thread (TQ * items per thread)

struct PwaParams {
  const float* q;           // [T, H*d]
  const void* cache;
  const int* block_tables;
  int max_blocks;
  const int* tiles;         // [n, 4] = (first token row, tokens, block-table row, 0)
  int tile_tokens;          // most tokens a tile can have
  const int* positions;
  const float* temp;        // [H] or null
  const float* talk;        // [H, H] or null
  float scale;
  int H, G, d, e, S, P, bs, PS, CG;
  void* out;                // [T, H*e]
};

template <typename T, int TQ>
__global__ void __launch_bounds__(256)
pooled_window_attention_kernel(const PwaParams p) {
  extern __shared__ float sm[];
  const int H = p.H, G = p.G, d = p.d, e = p.e, S = p.S, P = p.P, bs = p.bs, PS = p.PS, CG = p.CG;
  const int rep = H / G, Wc = G * (d + e);
  const int parts = (p.tile_tokens + TQ - 1) / TQ;
  const int tile = blockIdx.x / parts, part = blockIdx.x % parts;
  const int t0 = p.tiles[tile * 4] + part * TQ;
  const int nq = min(TQ, p.tiles[tile * 4 + 1] - part * TQ);
  if (nq <= 0) return;
  const int* table = p.block_tables + static_cast<long long>(p.tiles[tile * 4 + 2]) * p.max_blocks;
  const int p_first = p.positions[t0], p_last = p_first + nq - 1;
  const T* cache = static_cast<const T*>(p.cache);

  const int dmax = d > e ? d : e;
  const int kvld = CG * dmax + 1;
  float* Qs = sm;                                  // [H][d][TQ]
  float* KV = Qs + H * d * TQ;                     // [kTK][kvld]
  float* Pa = KV + kTK * kvld;                     // [H][kTK][TQ]   scores, then normalised weights
  float* Pb = Pa + H * kTK * TQ;                   // [H][kTK][TQ]   mixed weights
  float* sM = Pb + H * kTK * TQ;                   // [H][TQ]
  float* sL = sM + H * TQ;                         // [H][TQ]
  float* sTalk = sL + H * TQ;                      // [H][H]
  int* klo = reinterpret_cast<int*>(sTalk + H * H);   // [kTK]
  int* khi = klo + kTK;
  int* krow = khi + kTK;                           // cache row of each key (rows of Wc numbers)

  const int tid = threadIdx.x;
  for (int i = tid; i < H * d * TQ; i += 256) {
    const int qi = i % TQ, dd = (i / TQ) % d, h = i / (TQ * d);
    float v = 0.f;
    if (qi < nq) v = p.q[static_cast<long long>(t0 + qi) * H * d + h * d + dd] * (p.scale * (p.temp ? p.temp[h] : 1.f));
    Qs[i] = v;
  }
  for (int i = tid; i < H * TQ; i += 256) {
    sM[i] = -INFINITY;
    sL[i] = 0.f;
  }
  if (p.talk)
    for (int i = tid; i < H * H; i += 256) sTalk[i] = p.talk[i];

  // unified key list: pooled blocks 0..nb-1 (all seen by the last query), then tokens j0..p_last
  const int nb = (S > 0 && p_last - S + 1 >= P) ? (p_last - S + 1) / P : 0;
  const int j0 = (S > 0 && p_first - S + 1 > 0) ? p_first - S + 1 : 0;
  const int NU = nb + (p_last - j0 + 1);

  float acc[kAcc / TQ][TQ];
#pragma unroll
  for (int a = 0; a < kAcc / TQ; ++a)
#pragma unroll
    for (int qi = 0; qi < TQ; ++qi) acc[a][qi] = 0.f;

  for (int pass = 0; pass < 2; ++pass) {
    for (int u0 = 0; u0 < NU; u0 += kTK) {
      const int nk = min(kTK, NU - u0);
      __syncthreads();                                  // the previous tile is done with KV / Pa / Pb / key rows
      if (tid < kTK) {
        const int u = u0 + tid;
        int lo = INT_MAX, hi = INT_MIN;                 // an empty range: padding keys are seen by nobody
        int r = 0;
        if (u < nb) {
          lo = u * P + P - 1 + S;
          hi = INT_MAX;
          r = static_cast<int>(pooled_row(table, u, P, bs, PS));
        } else if (u < NU) {
          const int j = j0 + (u - nb);
          lo = j;
          hi = S > 0 ? j + S - 1 : INT_MAX;
          r = static_cast<int>(token_row(table, j, bs, PS));
        }
        klo[tid] = lo;
        khi[tid] = hi;
        krow[tid] = r;
      }
      __syncthreads();
      // ---- scores of every head for this key tile, one group of CG key heads at a time ----
      for (int c0 = 0; c0 < G; c0 += CG) {
        const int cg = min(CG, G - c0);
        if (c0 > 0) __syncthreads();
        for (int i = tid; i < kTK * cg * d; i += 256) {
          const int k = i / (cg * d), x = i % (cg * d);
          KV[k * kvld + x] = k < nk ? to_f32(cache[static_cast<long long>(krow[k]) * Wc + c0 * d + x]) : 0.f;
        }
        __syncthreads();
        for (int it = tid; it < cg * rep * kTK; it += 256) {
          const int k = it % kTK, hl = it / kTK;
          const int g = c0 * rep + hl, cl = hl / rep;
          float s[TQ];
#pragma unroll
          for (int qi = 0; qi < TQ; ++qi) s[qi] = 0.f;
          const float* kr = KV + k * kvld + cl * d;
          const float* qr = Qs + g * d * TQ;
          for (int dd = 0; dd < d; ++dd) {
            const float kv = kr[dd];
#pragma unroll
            for (int qi = 0; qi < TQ; ++qi) s[qi] = fmaf(qr[dd * TQ + qi], kv, s[qi]);
          }
          const int lo = klo[k], hi = khi[k];
#pragma unroll
          for (int qi = 0; qi < TQ; ++qi) {
            const int pi = p_first + qi;
            const bool seen = qi < nq && pi >= lo && pi <= hi;
            float v = seen ? s[qi] : -INFINITY;
            if (pass == 1) v = seen ? expf(v - sM[g * TQ + qi]) * sL[g * TQ + qi] : 0.f;
            Pa[(g * kTK + k) * TQ + qi] = v;
          }
        }
      }
      __syncthreads();
      if (pass == 0) {
        // ---- running maximum and sum of every (head, query) row ----
        for (int r = tid; r < H * TQ; r += 256) {
          const int g = r / TQ, qi = r % TQ;
          float m = sM[r], l = sL[r], tm = -INFINITY;
          for (int k = 0; k < kTK; ++k) tm = fmaxf(tm, Pa[(g * kTK + k) * TQ + qi]);
          if (tm > -INFINITY) {
            const float mn = fmaxf(m, tm);
            float add = 0.f;
            for (int k = 0; k < kTK; ++k) add += expf(Pa[(g * kTK + k) * TQ + qi] - mn);
            l = l * expf(m - mn) + add;              // exp(-inf) = 0 on the first tile that shows a key
            sM[r] = mn;
            sL[r] = l;
          }
        }
        continue;
      }
      // ---- pass 1: mix the normalised weights across heads ----
      const float* W = Pa;
      if (p.talk) {
        for (int i = tid; i < H * kTK * TQ; i += 256) {
          const int h = i / (kTK * TQ), rest = i % (kTK * TQ);
          float v = 0.f;
          for (int g = 0; g < H; ++g) v = fmaf(sTalk[h * H + g], Pa[g * kTK * TQ + rest], v);
          Pb[i] = v;
        }
        W = Pb;
      }
      // ---- values ----
      for (int c0 = 0; c0 < G; c0 += CG) {
        const int cg = min(CG, G - c0);
        __syncthreads();
        for (int i = tid; i < kTK * cg * e; i += 256) {
          const int k = i / (cg * e), x = i % (cg * e);
          KV[k * kvld + x] = k < nk ? to_f32(cache[static_cast<long long>(krow[k]) * Wc + G * d + c0 * e + x]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int a = 0; a < kAcc / TQ; ++a) {
          const int item = tid + a * 256;
          if (item >= H * e) break;
          const int h = item / e, col = item % e, c = h / rep;
          if (c < c0 || c >= c0 + cg) continue;
          const float* vr = KV + (c - c0) * e + col;
          const float* wr = W + h * kTK * TQ;
          for (int k = 0; k < kTK; ++k) {
            const float v = vr[k * kvld];
#pragma unroll
            for (int qi = 0; qi < TQ; ++qi) acc[a][qi] = fmaf(wr[k * TQ + qi], v, acc[a][qi]);
          }
        }
      }
    }
    if (pass == 0) {
      __syncthreads();
      for (int r = tid; r < H * TQ; r += 256) sL[r] = sL[r] > 0.f ? 1.f / sL[r] : 0.f;     // 1 / sum from here on
    }
  }
  T* out = static_cast<T*>(p.out);
#pragma unroll
  for (int a = 0; a < kAcc / TQ; ++a) {
    const int item = tid + a * 256;
    if (item >= H * e) break;
#pragma unroll
    for (int qi = 0; qi < TQ; ++qi)
      if (qi < nq) out[static_cast<long long>(t0 + qi) * H * e + item] = from_f32<T>(acc[a][qi]);
  }
}

static size_t pwa_smem_bytes(int H, int d, int e, int TQ, int CG) {
  const int dmax = d > e ? d : e;
  size_t fl = static_cast<size_t>(H) * d * TQ + static_cast<size_t>(kTK) * (CG * dmax + 1) + 2ull * H * kTK * TQ + 2ull * H * TQ +
              static_cast<size_t>(H) * H;
  return fl * 4 + 3 * kTK * 4;
}

template <typename T, int TQ>
static cudaError_t pwa_launch(const PwaParams& p, int ntiles, size_t smem, cudaStream_t s) {
  auto kern = pooled_window_attention_kernel<T, TQ>;
  cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (err != cudaSuccess) return err;
  const int parts = (p.tile_tokens + TQ - 1) / TQ;
  kern<<<ntiles * parts, 256, smem, s>>>(p);
  return cudaSuccess;
}

}  // namespace llmctl

using namespace llmctl;

// qkv: [tokens, H*d + G*d + G*e] (row stride ld) in the activation type; bias: same width or null; qn_w / kn_w: fp32
// norm weights over the whole q / k projection, or null for no norm; rot: rotated numbers per head (even, <= d), freq:
// fp32 [rot/2]; q_out: fp32 [tokens, H*d]; cache: [pages, bs + PS, G*(d+e)]; slots: int64 [tokens] = page * bs + offset
// (negative: the token is not cached); v_mode: 0 plain, 1 also store the values in v_first [tokens, G*e], 2 mix with
// v_first by lam (one fp32 number on the device).
LLMCTL_API int llmctl_window_qkv_write(const void* qkv, long long ld, const void* bias, const float* qn_w, const float* kn_w,
                                       int H, int G, int d, int e, int rot, const float* freq, float mult, float eps,
                                       const int* positions, const long long* slots, float* q_out, void* cache, int bs, int PS,
                                       void* v_first, int v_mode, const float* lam, int tokens, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0 && rot >= 0 && rot <= d && rot % 2 == 0 && bs > 0 && PS >= 0);
  LLMCTL_REQUIRE(v_mode == 0 || (v_first != nullptr && (v_mode == 1 || lam != nullptr)));
  if (tokens == 0) return 0;
  const size_t smem = static_cast<size_t>(H + G) * d * sizeof(float);
  LLMCTL_REQUIRE(smem <= 200 * 1024);
  cudaStream_t s = (cudaStream_t)stream;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, {
    auto kern = window_qkv_write_kernel<T>;
    if (smem > 48 * 1024) LLMCTL_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kern<<<tokens, 256, smem, s>>>((const T*)qkv, ld, (const T*)bias, qn_w, kn_w, H, G, d, e, rot, freq, mult, eps, positions, slots,
                                   q_out, (T*)cache, bs, PS, (T*)v_first, v_mode, lam);
  });
  LLMCTL_RETURN_LAST();
}

// seq_rows: int32 [tokens] = block-table row of each token's sequence; Wc = G*(d+e).
LLMCTL_API int llmctl_window_pool_update(void* cache, const int* positions, const long long* slots, const int* seq_rows,
                                         const int* block_tables, int max_blocks, int bs, int PS, int P, int Wc, int tokens,
                                         int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(P > 0 && bs > 0 && PS == (bs + P - 1) / P && Wc > 0);
  if (tokens == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (window_pool_update_kernel<T><<<tokens, 128, 0, (cudaStream_t)stream>>>(
      (T*)cache, positions, slots, seq_rows, block_tables, max_blocks, bs, PS, P, Wc)));
  LLMCTL_RETURN_LAST();
}

// The most tokens per CTA (1, 2, 4, 8 or 16, at most tile_tokens) whose accumulators and shared memory fit; 0 if
// even one token does not.
LLMCTL_API int llmctl_pooled_window_attention_rows(int H, int d, int e, int tile_tokens) {
  for (int tq = 16; tq >= 1; tq >>= 1) {
    if (tq > 1 && tq > tile_tokens) continue;
    if (((H * e + 255) / 256) * tq > kAcc) continue;
    if (pwa_smem_bytes(H, d, e, tq, 1) > 160 * 1024) continue;
    return tq;
  }
  return 0;
}

// q: fp32 [tokens, H*d]; tiles: int32 [ntiles, 4] = (first token row, tokens <= tile_tokens, block-table row, 0), the
// tokens of a tile being consecutive positions of one sequence; S: window (0 = every earlier token, no pooling);
// P: pool; temp: fp32 [H] or null; talk: fp32 [H, H] or null; out: [tokens, H*e] in the cache's type.
LLMCTL_API int llmctl_pooled_window_attention(const float* q, const void* cache, const int* block_tables, int max_blocks,
                                              const int* tiles, int ntiles, int tile_tokens, const int* positions,
                                              const float* temp, const float* talk, float scale, int H, int G, int d, int e,
                                              int S, int P, int bs, int PS, void* out, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0 && S >= 0 && (S == 0 || P > 0) && bs > 0 && tile_tokens > 0);
  if (ntiles == 0) return 0;
  const int TQ = llmctl_pooled_window_attention_rows(H, d, e, tile_tokens);
  LLMCTL_REQUIRE(TQ > 0);
  int CG = 1;
  while (CG < G && pwa_smem_bytes(H, d, e, TQ, CG + 1) <= 96 * 1024) ++CG;
  PwaParams p{q, cache, block_tables, max_blocks, tiles, tile_tokens, positions, temp, talk, scale, H, G, d, e, S, P, bs, PS, CG, out};
  const size_t smem = pwa_smem_bytes(H, d, e, TQ, CG);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t err = cudaSuccess;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, {
    switch (TQ) {
      case 16: err = pwa_launch<T, 16>(p, ntiles, smem, s); break;
      case 8: err = pwa_launch<T, 8>(p, ntiles, smem, s); break;
      case 4: err = pwa_launch<T, 4>(p, ntiles, smem, s); break;
      case 2: err = pwa_launch<T, 2>(p, ntiles, smem, s); break;
      default: err = pwa_launch<T, 1>(p, ntiles, smem, s); break;
    }
  });
  if (err != cudaSuccess) LLMCTL_FAIL(err, "attribute");
  LLMCTL_RETURN_LAST();
}
