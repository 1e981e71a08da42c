// Paged causal attention over the cache for any mix of rows: one warp per (row, query head).
//   s_p = dot(q, K[p]) * scale for the keys p of the row's own request with lo <= p <= pos,
//   lo = first_key(pos, window) (a sliding window, or the query's own chunk); softmax and the weighted sum of V in
//   32-bit with a running maximum.
// Keys are visited in tiles of 32 aligned to absolute positions, each lane scoring one key, so
// the order of every sum depends only on positions: the result for a row is the same however the
// tokens were cut into steps, whatever else is in the batch and whichever pages hold the keys.
// Any head size up to 640 (multiples of 8 are read in wide pieces); any number of heads and groups.
// Two options: `sink`, a number per query head that is added to the softmax's sum as exp(sink)
// (a key that has no value: it takes weight and gives nothing); `vd`, how many of a value
// row's first channels are summed and written (out is [rows][Hq][vd]; the rest of a value row is
// not read), for caches whose values are a prefix of their keys.
// Two more: `keep_first`, the first so many keys of a sequence are seen from every later position
// although a window has passed them; and a second, pooled cache (`pool` > 0) that holds one key
// and value per block of `pool` positions, of which a row sees the blocks that end at or before
// pos - window.  Pooled blocks, kept keys, the window's keys and the sink share one softmax; they
// are visited in that order, in tiles of 32 aligned to entry 0 and to absolute positions.
#include "common.cuh"

namespace {
constexpr int MAX_HD = 640;
constexpr int WARPS = 4;

template <typename T> struct Vec8;  // 8 elements of T loaded at once
template <> struct Vec8<float> {
  float v[8];
  __device__ __forceinline__ void load(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct Vec8<bf16> {
  float v[8];
  __device__ __forceinline__ void load(const bf16* p) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// VEC: the head size is a multiple of 8, so a key row is read in 16-byte (32-byte) pieces.
// NACC: 32-channel pieces of a value row that a lane sums (vd <= 32 * NACC)
// the second cache of a layer with pooled blocks (null k: none)
struct PooledSource {
  const void *k, *v;
  long long page_stride;
  const int* table;
  int table_stride, pool;
};

// VEC: the head size is a multiple of 8, so a key row is read in 16-byte (32-byte) pieces.
// NACC: 32-channel pieces of a value row that a lane sums (vd <= 32 * NACC)
// EXTRAS: only what lies outside the window (pooled blocks, kept first keys, the sink) is summed,
// and the result is left as a part for a merge with the window's keys, which another kernel sums:
// part_o [rows][Hq][hd] the weighted values without the division, part_ml [rows][Hq][2] the
// maximum as a base-2 logarithm (score times log2 e) and the sum of the weights.
template <typename T, bool VEC, int NACC, bool EXTRAS>
__global__ void __launch_bounds__(WARPS * 32) attention_generic_kernel(
    const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, long long page_stride, const int* __restrict__ block_table,
    int table_stride, const int* __restrict__ row_slot, const int* __restrict__ row_pos, int rows,
    int Hq, int Hkv, int hd, int page_size, float scale, int window, const float* __restrict__ sink, int vd,
    int keep_first, const PooledSource pooled, float* __restrict__ part_o, float* __restrict__ part_ml) {
  __shared__ float q_s[WARPS][MAX_HD];
  const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp_in_block;
  if (item >= (long long)rows * Hq) return;
  const int t = (int)(item / Hq), h = (int)(item % Hq);
  const int kvh = h / (Hq / Hkv);
  const int pos = row_pos[t];
  const int* table = block_table + (size_t)row_slot[t] * table_stride;
  const int lo = first_key(pos, window);

  float* qs = q_s[warp_in_block];
  const T* qrow = q + ((size_t)t * Hq + h) * hd;
  for (int i = lane; i < hd; i += 32) qs[i] = to_f32(qrow[i]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;

  // one tile: this lane's entry is visible or not; kc / vc and off say where its rows lie
  auto tile = [&](bool valid, const T* kc, const T* vc, long long off) {
    float s = -INFINITY;
    if (valid) {
      const T* kr = kc + off;
      float d = 0.f;
      if (VEC) {
        for (int i = 0; i < hd; i += 8) {
          Vec8<T> kv;
          kv.load(kr + i);
#pragma unroll
          for (int j = 0; j < 8; ++j) d = fmaf(qs[i + j], kv.v[j], d);
        }
      } else {
        for (int i = 0; i < hd; ++i) d = fmaf(qs[i], to_f32(kr[i]), d);
      }
      s = d * scale;
    }
    const unsigned mask = __ballot_sync(0xffffffffu, valid);
    if (mask == 0) return;
    const float m_new = fmaxf(m, warp_max(s));
    const float w = valid ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(w);
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] *= corr;
    m = m_new;
    for (int j = 0; j < 32; ++j) {
      if (!((mask >> j) & 1u)) continue;
      const float wj = __shfl_sync(0xffffffffu, w, j);
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      const T* vr = vc + oj;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) acc[i] = fmaf(wj, to_f32(vr[d]), acc[i]);
      }
    }
  };

  if (pooled.k != nullptr && window > 0) {
    // blocks b with b * pool + pool - 1 <= pos - window
    const int seen = pos - window + 1 >= pooled.pool ? (pos - window + 1) / pooled.pool : 0;
    const int* ptable = pooled.table + (size_t)row_slot[t] * pooled.table_stride;
    for (int base = 0; base < seen; base += 32) {
      const int b = base + lane;
      const bool valid = b < seen;
      long long off = 0;
      if (valid)
        off = (long long)ptable[b / page_size] * pooled.page_stride +
              ((long long)kvh * page_size + b % page_size) * hd;
      tile(valid, (const T*)pooled.k, (const T*)pooled.v, off);
    }
  }
  // the kept first keys that the window has passed (those inside it are met below)
  const int kept = keep_first < lo ? keep_first : lo;
  for (int base = 0; base < kept; base += 32) {
    const int p = base + lane;
    const bool valid = p < kept;
    long long off = 0;
    if (valid)
      off = (long long)table[p / page_size] * page_stride + ((long long)kvh * page_size + p % page_size) * hd;
    tile(valid, k_cache, v_cache, off);
  }
  if (EXTRAS) {
    if (sink) {      // the sink is one more entry of this part
      const float m_new = fmaxf(m, sink[h]);
      const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
      l = l * corr + expf(sink[h] - m_new);
#pragma unroll
      for (int i = 0; i < NACC; ++i) acc[i] *= corr;
      m = m_new;
    }
    float* po = part_o + ((size_t)t * Hq + h) * hd;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) po[d] = d < vd ? acc[i] : 0.f;
    }
    if (lane == 0) {
      part_ml[((size_t)t * Hq + h) * 2] = m * 1.4426950408889634f;
      part_ml[((size_t)t * Hq + h) * 2 + 1] = l;
    }
    return;
  }
  for (int base = (lo / 32) * 32; base <= pos; base += 32) {
    const int p = base + lane;
    const bool valid = p >= lo && p <= pos;
    long long off = 0;  // element offset of this lane's key row inside the layer's cache
    if (valid)
      off = (long long)table[p / page_size] * page_stride + ((long long)kvh * page_size + p % page_size) * hd;
    tile(valid, k_cache, v_cache, off);
  }
  if (sink) l += expf(sink[h] - m);     // (m is finite: a row sees at least its own key)
  const float inv = 1.0f / l;
  T* orow = out + ((size_t)t * Hq + h) * vd;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < vd) orow[d] = from_f32<T>(acc[i] * inv);
  }
}

// What lies outside the window for all heads of a group at once: one warp per (row, key head).
// A lane scores one entry (a pooled block or a kept first key) against the GROUP queries that
// share it, so a key row is read once for the group; the values are summed with a lane per pair
// of channels.  Head sizes 64 and 128, bfloat16, 16-byte aligned rows.  The result is one part
// per row and query head, as the EXTRAS form of the kernel above leaves it.
template <int GROUP>
__global__ void __launch_bounds__(WARPS * 32) attention_outside_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    long long page_stride, const int* __restrict__ block_table, int table_stride, const int* __restrict__ row_slot,
    const int* __restrict__ row_pos, int rows, int Hq, int Hkv, int hd, int page_size, float scale, int window,
    const float* __restrict__ sink, int keep_first, const PooledSource pooled, float* __restrict__ part_o,
    float* __restrict__ part_ml) {
  __shared__ __align__(16) float q_s[WARPS][GROUP][128];
  const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // (the warps of a block are adjacent rows on one key head: in a prompt's portion they read the
  // same entries at about the same time, which the first-level cache then serves)
  const int t = blockIdx.x * WARPS + warp_in_block, kvh = blockIdx.y;
  if (t >= rows) return;
  const int pos = row_pos[t], slot = row_slot[t];
  const int* table = block_table + (size_t)slot * table_stride;
  const int behind = pos - window + 1 > 0 ? pos - window + 1 : 0;      // positions the window has passed
  const int kept = keep_first < behind ? keep_first : behind;
  const int seen = pooled.k != nullptr ? behind / pooled.pool : 0;     // blocks that lie wholly behind it
  const int* ptable = pooled.k != nullptr ? pooled.table + (size_t)slot * pooled.table_stride : nullptr;
  const int total = seen + kept;
  const int pairs = hd / 64;      // pairs of channels per lane

  float (*qs)[128] = q_s[warp_in_block];
  const bf16* qrow = q + ((size_t)t * Hq + (size_t)kvh * GROUP) * hd;
  for (int i = lane; i < GROUP * hd; i += 32) qs[i / hd][i % hd] = to_f32(qrow[i]);
  __syncwarp();

  float m[GROUP], l[GROUP], acc[GROUP][4];
#pragma unroll
  for (int g = 0; g < GROUP; ++g) {
    m[g] = -INFINITY, l[g] = 0.f;
    acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
  }
  for (int base = 0; base < total; base += 32) {
    const int e = base + lane;
    const bool valid = e < total;
    const bf16 *kr = k_cache, *vr = v_cache;
    if (valid) {
      if (e < seen) {
        const long long off = (long long)ptable[e / page_size] * pooled.page_stride +
                              ((long long)kvh * page_size + e % page_size) * hd;
        kr = (const bf16*)pooled.k + off, vr = (const bf16*)pooled.v + off;
      } else {
        const int p = e - seen;
        const long long off = (long long)table[p / page_size] * page_stride +
                              ((long long)kvh * page_size + p % page_size) * hd;
        kr = k_cache + off, vr = v_cache + off;
      }
    }
    float w[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) w[g] = 0.f;
    if (valid) {
#pragma unroll 4
      for (int i = 0; i < hd; i += 8) {
        Vec8<bf16> kv;
        kv.load(kr + i);
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
          const float4 a = *reinterpret_cast<const float4*>(&qs[g][i]);
          const float4 b = *reinterpret_cast<const float4*>(&qs[g][i + 4]);
          float d = w[g];
          d = fmaf(a.x, kv.v[0], d), d = fmaf(a.y, kv.v[1], d), d = fmaf(a.z, kv.v[2], d), d = fmaf(a.w, kv.v[3], d);
          d = fmaf(b.x, kv.v[4], d), d = fmaf(b.y, kv.v[5], d), d = fmaf(b.z, kv.v[6], d), d = fmaf(b.w, kv.v[7], d);
          w[g] = d;
        }
      }
    }
    const unsigned mask = __ballot_sync(0xffffffffu, valid);
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const float sc = valid ? w[g] * scale : -INFINITY;
      const float m_new = fmaxf(m[g], warp_max(sc));
      w[g] = valid ? expf(sc - m_new) : 0.f;
      const float corr = (m[g] == -INFINITY) ? 0.f : expf(m[g] - m_new);
      l[g] = l[g] * corr + warp_sum(w[g]);
      acc[g][0] *= corr, acc[g][1] *= corr, acc[g][2] *= corr, acc[g][3] *= corr;
      m[g] = m_new;
    }
    const int nv = __popc(mask);      // the entries of a tile are its first lanes
    for (int j0 = 0; j0 < nv; j0 += 4) {
      // four value rows at a time: their loads are under way together
      float2 v0[4], v1[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bf16* vj = (const bf16*)__shfl_sync(0xffffffffu, (unsigned long long)vr, (j0 + i) & 31);
        v0[i] = v1[i] = make_float2(0.f, 0.f);
        if (j0 + i < nv) {
          const uint32_t a = *reinterpret_cast<const uint32_t*>(vj + 2 * lane);
          v0[i] = make_float2(__uint_as_float(a << 16), __uint_as_float(a & 0xffff0000u));
          if (pairs > 1) {
            const uint32_t b = *reinterpret_cast<const uint32_t*>(vj + 64 + 2 * lane);
            v1[i] = make_float2(__uint_as_float(b << 16), __uint_as_float(b & 0xffff0000u));
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
          // (a lane behind the tile's entries has the weight 0 and met zeros above)
          const float wj = __shfl_sync(0xffffffffu, w[g], (j0 + i) & 31);
          acc[g][0] = fmaf(wj, v0[i].x, acc[g][0]), acc[g][1] = fmaf(wj, v0[i].y, acc[g][1]);
          acc[g][2] = fmaf(wj, v1[i].x, acc[g][2]), acc[g][3] = fmaf(wj, v1[i].y, acc[g][3]);
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < GROUP; ++g) {
    const int h = kvh * GROUP + g;
    float mg = m[g], lg = l[g], corr = 1.f;
    if (sink) {      // the sink is one more entry of this part
      const float m_new = fmaxf(mg, sink[h]);
      corr = (mg == -INFINITY) ? 0.f : expf(mg - m_new);
      lg = lg * corr + expf(sink[h] - m_new);
      mg = m_new;
    }
    float* po = part_o + ((size_t)t * Hq + h) * hd;
    *reinterpret_cast<float2*>(po + 2 * lane) = make_float2(acc[g][0] * corr, acc[g][1] * corr);
    if (pairs > 1) *reinterpret_cast<float2*>(po + 64 + 2 * lane) = make_float2(acc[g][2] * corr, acc[g][3] * corr);
    if (lane == 0) {
      part_ml[((size_t)t * Hq + h) * 2] = mg * 1.4426950408889634f;
      part_ml[((size_t)t * Hq + h) * 2 + 1] = lg;
    }
  }
}
}  // namespace

// keep_first and the pooled cache (pk_cache null: none) as described at the top of this file
LLM_EXPORT int llm_attention_generic_ext(const void* q, void* out, const void* k_cache, const void* v_cache,
                                         int dtype, long long page_stride, const int* block_table,
                                         int table_stride, const int* row_slot, const int* row_pos, int rows,
                                         int Hq, int Hkv, int hd, int page_size, float scale, int window,
                                         const float* sink, int vd, int keep_first, const void* pk_cache,
                                         const void* pv_cache, long long p_page_stride, const int* p_table,
                                         int p_table_stride, int pool, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vd <= 0) vd = hd;
  if (hd > MAX_HD || hd <= 0 || vd > hd || Hkv <= 0 || Hq % Hkv != 0) return LLM_ERR_UNSUPPORTED;
  if (keep_first < 0 || (pk_cache != nullptr && (pool <= 0 || window <= 0 || !pv_cache || !p_table)))
    return LLM_ERR_ARGUMENT;
  PooledSource pooled;
  pooled.k = pk_cache, pooled.v = pv_cache, pooled.page_stride = p_page_stride, pooled.table = p_table;
  pooled.table_stride = p_table_stride, pooled.pool = pool;
  const bool vec = hd % 8 == 0 && (page_stride % 8) == 0 &&
                   (((uintptr_t)k_cache | (uintptr_t)v_cache) & 31) == 0 &&
                   (pk_cache == nullptr ||
                    ((p_page_stride % 8) == 0 && (((uintptr_t)pk_cache | (uintptr_t)pv_cache) & 31) == 0));
  const long long items = (long long)rows * Hq;
  const int blocks = (int)((items + WARPS - 1) / WARPS);
#define GENERIC(T, V, N)                                                                            \
  attention_generic_kernel<T, V, N, false><<<blocks, WARPS * 32, 0, stream>>>(                      \
      (const T*)q, (T*)out, (const T*)k_cache, (const T*)v_cache, page_stride, block_table,         \
      table_stride, row_slot, row_pos, rows, Hq, Hkv, hd, page_size, scale, window, sink, vd,       \
      keep_first, pooled, nullptr, nullptr)
#define GENERIC_N(T, V)                                  \
  do {                                                   \
    if (vd <= 128) GENERIC(T, V, 4);                     \
    else if (vd <= 256) GENERIC(T, V, 8);                \
    else GENERIC(T, V, MAX_HD / 32);                     \
  } while (0)
  if (dtype == LLM_F32) {
    if (vec) GENERIC_N(float, true); else GENERIC_N(float, false);
  } else if (dtype == LLM_BF16) {
    if (vec) GENERIC_N(bf16, true); else GENERIC_N(bf16, false);
  } else {
    return LLM_ERR_UNSUPPORTED;
  }
#undef GENERIC_N
#undef GENERIC
  return launch_status();
}

LLM_EXPORT int llm_attention_generic(const void* q, void* out, const void* k_cache,
                                     const void* v_cache, int dtype, long long page_stride,
                                     const int* block_table, int table_stride, const int* row_slot,
                                     const int* row_pos, int rows, int Hq, int Hkv, int hd,
                                     int page_size, float scale, int window, const float* sink, int vd,
                                     cudaStream_t stream) {
  return llm_attention_generic_ext(q, out, k_cache, v_cache, dtype, page_stride, block_table, table_stride,
                                   row_slot, row_pos, rows, Hq, Hkv, hd, page_size, scale, window, sink, vd, 0,
                                   nullptr, nullptr, 0, nullptr, 0, 0, stream);
}

// Only what a row sees outside its window: the pooled blocks that lie behind it, the kept first
// keys that it has passed, and the sink, as one part for a merge with the window's keys (which the
// tensor-core kernels sum).  bfloat16 caches with head sizes up to 128 that are multiples of 8.
LLM_EXPORT int llm_attention_extras(const void* q, float* part_o, float* part_ml, const void* k_cache,
                                    const void* v_cache, long long page_stride, const int* block_table,
                                    int table_stride, const int* row_slot, const int* row_pos, int rows, int Hq,
                                    int Hkv, int hd, int page_size, float scale, int window, const float* sink,
                                    int keep_first, const void* pk_cache, const void* pv_cache,
                                    long long p_page_stride, const int* p_table, int p_table_stride, int pool,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hd > 128 || hd <= 0 || hd % 8 || Hkv <= 0 || Hq % Hkv != 0 || window <= 0) return LLM_ERR_UNSUPPORTED;
  if (keep_first < 0 || !part_o || !part_ml || (pk_cache != nullptr && (pool <= 0 || !pv_cache || !p_table)))
    return LLM_ERR_ARGUMENT;
  PooledSource pooled;
  pooled.k = pk_cache, pooled.v = pv_cache, pooled.page_stride = p_page_stride, pooled.table = p_table;
  pooled.table_stride = p_table_stride, pooled.pool = pool;
  const bool vec = (page_stride % 8) == 0 && (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0 &&
                   (pk_cache == nullptr ||
                    ((p_page_stride % 8) == 0 && (((uintptr_t)pk_cache | (uintptr_t)pv_cache) & 15) == 0));
  const int group = Hq / Hkv;
  if (vec && (hd == 64 || hd == 128) && ((uintptr_t)q & 15) == 0 && ((uintptr_t)part_o & 7) == 0) {
    if (Hkv > 65535) return LLM_ERR_UNSUPPORTED;
    const dim3 nb((rows + WARPS - 1) / WARPS, Hkv);
#define OUTSIDE_GO(G)                                                                                          \
  attention_outside_kernel<G><<<nb, WARPS * 32, 0, stream>>>(                                                  \
      (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, block_table, table_stride,      \
      row_slot, row_pos, rows, Hq, Hkv, hd, page_size, scale, window, sink, keep_first, pooled, part_o, part_ml)
    switch (group) {
      case 1: OUTSIDE_GO(1); return launch_status();
      case 2: OUTSIDE_GO(2); return launch_status();
      case 4: OUTSIDE_GO(4); return launch_status();
      case 8: OUTSIDE_GO(8); return launch_status();
      case 16: OUTSIDE_GO(16); return launch_status();
      default: break;
    }
#undef OUTSIDE_GO
  }
  const long long items = (long long)rows * Hq;
  const int blocks = (int)((items + WARPS - 1) / WARPS);
#define EXTRAS_GO(V)                                                                                          \
  attention_generic_kernel<bf16, V, 4, true><<<blocks, WARPS * 32, 0, stream>>>(                              \
      (const bf16*)q, nullptr, (const bf16*)k_cache, (const bf16*)v_cache, page_stride, block_table,          \
      table_stride, row_slot, row_pos, rows, Hq, Hkv, hd, page_size, scale, window, sink, hd, keep_first,     \
      pooled, part_o, part_ml)
  if (vec) EXTRAS_GO(true);
  else EXTRAS_GO(false);
#undef EXTRAS_GO
  return launch_status();
}
