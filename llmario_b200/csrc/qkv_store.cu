// Queries, keys and values from their projections into the form attention reads, for mixers whose
// norm or rotation the per-head kernel (rope_kv.cu) does not have, and the pooled entries of a
// cache that keeps one key and value per block of tokens.
//
// llm_qkv_store, one block per row, a warp per head:
//   norm 0: none;  1: every head of q and k over its own `d` channels with a weight [d] shared by
//   the heads;  2: the whole q row (Hq * d channels) and the whole k row at once, weights of
//   that size.  All of it x * rsqrt(mean(x^2) + eps) * w in 32-bit.
//   rotation: the pairs (2i, 2i + 1), i < rot / 2, of every q and k head are turned by the row's
//   angles (cos and sin per (row, i) made once per step); the other channels pass.
//   q goes out as [rows][Hq][hd] in the step's type, keys and values into the pages of the row's
//   request; hd >= max(d, dv) is the cache's row, the channels behind d (dv) are written as zeros.
//   temperature: the queries of position p are multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).
//   blend: the value that is stored is (1 - lambda) v + lambda v0, v0 another layer's values of
//   the same rows (32-bit, as projected).
//
// llm_pool_blocks, one block per (row, key head): a row whose position ends a block of P tokens
// (pos % P == P - 1) writes entry pos / P of the pooled cache: the means of the block's P cached
// keys and of its P cached values, summed in 32-bit in ascending position.
#include "common.cuh"

namespace {

struct StoreArgs {
  const float *q, *k, *v;          // [rows][Hq * d], [rows][Hkv * d], [rows][Hkv * dv]
  int q_stride, k_stride, v_stride;
  const float *q_w, *k_w;
  const float* cos_sin;            // [rows][rot / 2][2] or null
  void* q_out;
  void *k_cache, *v_cache;
  long long page_stride;
  const int *table, *row_slot, *row_pos;
  int table_stride, page_size;
  int rows, Hq, Hkv, d, dv, hd, rot, norm, has_kv;
  float eps;
  float temp_coef; int temp_every;     // query temperature by position (every 0: none)
  const float* v0; int v0_stride;      // values to blend in ([rows][Hkv * dv]) or null
  float blend;
};

__device__ __forceinline__ void store2(float* dst, float a, float b) { *reinterpret_cast<float2*>(dst) = make_float2(a, b); }
__device__ __forceinline__ void store2(bf16* dst, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a, b);
}

// One block per (row, share of the heads); a warp per head in turn.  With a norm over whole rows
// every block of a row sums the squares of the whole row itself.  PAIRS: all sizes are even and
// the rows 8-byte aligned, so a lane reads and writes two adjacent channels at once, which are
// also the two members of a rotated pair.
template <typename T, bool PAIRS>
__global__ void __launch_bounds__(256) qkv_store_kernel(const StoreArgs a) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const float* qr = a.q + (size_t)r * a.q_stride;
  const float* kr = a.has_kv ? a.k + (size_t)r * a.k_stride : nullptr;
  float whole_q = 1.f, whole_k = 1.f;
  if (a.norm == 2) {
    float s = 0.f;
    if (PAIRS) {
      for (int i = threadIdx.x; i < a.Hq * a.d / 2; i += blockDim.x) {
        const float2 x = *reinterpret_cast<const float2*>(qr + 2 * i);
        s = fmaf(x.x, x.x, s), s = fmaf(x.y, x.y, s);
      }
    } else {
      for (int i = threadIdx.x; i < a.Hq * a.d; i += blockDim.x) s = fmaf(qr[i], qr[i], s);
    }
    whole_q = rsqrtf(block_sum(s, scratch) / (float)(a.Hq * a.d) + a.eps);
    if (a.has_kv) {
      s = 0.f;
      for (int i = threadIdx.x; i < a.Hkv * a.d; i += blockDim.x) s = fmaf(kr[i], kr[i], s);
      whole_k = rsqrtf(block_sum(s, scratch) / (float)(a.Hkv * a.d) + a.eps);
    }
  }
  const int pos = a.row_pos[r];
  const float temp = a.temp_every > 0
      ? 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every + 1)) : 1.f;
  long long page_off = 0;
  if (a.has_kv) {
    const int page = a.table[(size_t)a.row_slot[r] * a.table_stride + pos / a.page_size];
    page_off = (long long)page * a.page_stride;
  }
  const float* cs = a.cos_sin ? a.cos_sin + (size_t)r * (a.rot / 2) * 2 : nullptr;
  const int heads = a.Hq + (a.has_kv ? 2 * a.Hkv : 0);
  for (int item = blockIdx.y * nwarps + warp; item < heads; item += nwarps * gridDim.y) {
    if (item >= a.Hq + a.Hkv) {                    // a value head: a copy, padded with zeros
      const int g = item - a.Hq - a.Hkv;
      const float* src = a.v + (size_t)r * a.v_stride + (size_t)g * a.dv;
      const float* mix = a.v0 ? a.v0 + (size_t)r * a.v0_stride + (size_t)g * a.dv : nullptr;
      const float keep = 1.f - a.blend;
      T* dst = (T*)a.v_cache + page_off + ((long long)g * a.page_size + pos % a.page_size) * a.hd;
      if (PAIRS && !mix) {
        for (int c = 2 * lane; c < a.hd; c += 64) {
          float2 x = make_float2(0.f, 0.f);
          if (c < a.dv) x = *reinterpret_cast<const float2*>(src + c);
          store2(dst + c, x.x, x.y);
        }
      } else {
        for (int c = lane; c < a.hd; c += 32) {
          float x = c < a.dv ? src[c] : 0.f;
          if (mix && c < a.dv) x = fmaf(a.blend, mix[c], keep * x);
          dst[c] = from_f32<T>(x);
        }
      }
      continue;
    }
    const bool is_q = item < a.Hq;
    const int h = is_q ? item : item - a.Hq;
    const float* src = (is_q ? qr : kr) + (size_t)h * a.d;
    const float* w = is_q ? a.q_w : a.k_w;
    float scale = is_q ? whole_q : whole_k;
    if (a.norm == 1) {
      float s = 0.f;
      for (int c = lane; c < a.d; c += 32) s = fmaf(src[c], src[c], s);
      scale = rsqrtf(warp_sum(s) / (float)a.d + a.eps);
    }
    if (is_q) scale *= temp;
    if (w && a.norm == 2) w += (size_t)h * a.d;
    if (!a.norm) w = nullptr;
    T* dst = is_q ? (T*)a.q_out + ((size_t)r * a.Hq + h) * a.hd
                  : (T*)a.k_cache + page_off + ((long long)h * a.page_size + pos % a.page_size) * a.hd;
    if (PAIRS) {
      for (int c = 2 * lane; c < a.hd; c += 64) {
        float x = 0.f, y = 0.f;
        if (c < a.d) {
          const float2 u = *reinterpret_cast<const float2*>(src + c);
          x = u.x * scale * (w ? w[c] : 1.f);
          y = u.y * scale * (w ? w[c + 1] : 1.f);
          if (cs && c < a.rot) {
            const float2 t = *reinterpret_cast<const float2*>(cs + c);      // (cos, sin) of pair c / 2
            const float x2 = fmaf(x, t.x, -(y * t.y));
            y = fmaf(y, t.x, x * t.y);
            x = x2;
          }
        }
        store2(dst + c, x, y);
      }
      continue;
    }
    for (int c = lane; c < a.hd; c += 32) {
      float x = 0.f;
      if (c < a.d) {
        x = src[c] * scale * (w ? w[c] : 1.f);
        if (cs && c < a.rot) {
          const int o = c ^ 1;                       // the other member of the pair
          const float y = src[o] * scale * (w ? w[o] : 1.f);
          const float co = cs[(c >> 1) * 2], si = cs[(c >> 1) * 2 + 1];
          x = (c & 1) ? fmaf(x, co, y * si) : fmaf(x, co, -(y * si));
        }
      }
      dst[c] = from_f32<T>(x);
    }
  }
}

// A block per (row that ends a block of P positions, key head): `subs` groups of hd threads share
// out the block's positions (group s takes s, s + subs, ...), a thread per channel sums its
// group's keys and values, and the groups' sums are added in order through shared memory.  Which
// positions a sum visits in which order depends on P, hd and subs only.
template <typename T>
__global__ void __launch_bounds__(1024) pool_blocks_kernel(
    const T* __restrict__ k_cache, const T* __restrict__ v_cache, long long page_stride,
    const int* __restrict__ table, int table_stride, T* __restrict__ pk_cache, T* __restrict__ pv_cache,
    long long p_page_stride, const int* __restrict__ p_table, int p_table_stride, const int* __restrict__ row_slot,
    const int* __restrict__ row_pos, int Hkv, int hd, int page_size, int P, int subs) {
  extern __shared__ float sums[];      // [subs][2][hd]
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, g = blockIdx.y;
  const int pos = row_pos[r];
  if (pos % P != P - 1) return;
  const int b = pos / P, slot = row_slot[r];
  const int* tab = table + (size_t)slot * table_stride;
  const int sub = threadIdx.x / hd, c = threadIdx.x % hd;
  if (sub < subs) {
    float sk = 0.f, sv = 0.f;
    int p = b * P + sub;
    int page = p / page_size, in = p % page_size;
#pragma unroll 4
    for (int j = sub; j < P; j += subs) {
      const long long off = (long long)tab[page] * page_stride + ((long long)g * page_size + in) * hd + c;
      sk += to_f32(k_cache[off]);
      sv += to_f32(v_cache[off]);
      in += subs;
      while (in >= page_size) in -= page_size, ++page;
    }
    sums[(sub * 2) * hd + c] = sk, sums[(sub * 2 + 1) * hd + c] = sv;
  }
  __syncthreads();
  if (sub != 0) return;
  float sk = 0.f, sv = 0.f;
  for (int s = 0; s < subs; ++s) sk += sums[(s * 2) * hd + c], sv += sums[(s * 2 + 1) * hd + c];
  const int dst_page = p_table[(size_t)slot * p_table_stride + b / page_size];
  const long long dst = (long long)dst_page * p_page_stride + ((long long)g * page_size + b % page_size) * hd;
  const float inv = 1.0f / (float)P;
  pk_cache[dst + c] = from_f32<T>(sk * inv);
  pv_cache[dst + c] = from_f32<T>(sv * inv);
}
}  // namespace

LLM_EXPORT int llm_qkv_store_mix(const float* q, int q_stride, const float* k, int k_stride, const float* v,
                                 int v_stride, const float* q_w, const float* k_w, const float* cos_sin,
                                 void* q_out, void* k_cache, void* v_cache, int dtype, long long page_stride,
                                 const int* table, int table_stride, const int* row_slot, const int* row_pos,
                                 int rows, int Hq, int Hkv, int d, int dv, int hd, int rot, int norm, float eps,
                                 int page_size, int has_kv, float temp_coef, int temp_every, const float* v0,
                                 int v0_stride, float blend, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (temp_every < 0) return LLM_ERR_ARGUMENT;
  if (d <= 0 || dv <= 0 || hd < d || hd < dv || rot < 0 || rot > d || (rot & 1) || norm < 0 || norm > 2)
    return LLM_ERR_ARGUMENT;
  if (rot > 0 && !cos_sin) return LLM_ERR_ARGUMENT;
  StoreArgs a;
  a.q = q, a.k = k, a.v = v, a.q_stride = q_stride, a.k_stride = k_stride, a.v_stride = v_stride;
  a.q_w = q_w, a.k_w = k_w, a.cos_sin = rot > 0 ? cos_sin : nullptr, a.q_out = q_out, a.k_cache = k_cache,
  a.v_cache = v_cache;
  a.page_stride = page_stride, a.table = table, a.row_slot = row_slot, a.row_pos = row_pos;
  a.table_stride = table_stride, a.page_size = page_size, a.rows = rows, a.Hq = Hq, a.Hkv = Hkv, a.d = d,
  a.dv = dv, a.hd = hd, a.rot = rot, a.norm = norm, a.has_kv = has_kv, a.eps = eps;
  a.temp_coef = temp_coef, a.temp_every = temp_every, a.v0 = has_kv ? v0 : nullptr, a.v0_stride = v0_stride,
  a.blend = blend;
  const int heads = Hq + (has_kv ? 2 * Hkv : 0);
  const int threads = heads >= 8 ? 256 : heads >= 4 ? 128 : 64;
  // few rows: the heads of a row are shared out to several blocks, so that the step fills the GPU
  int shares = 1;
  if (rows < 1024) {
    shares = (heads + threads / 32 - 1) / (threads / 32);
    if (shares > 8) shares = 8;
  }
  const bool even = !((d | dv | hd | q_stride) & 1) && !((uintptr_t)q & 7) && !((uintptr_t)q_out & 7) &&
                    (!has_kv || (!((k_stride | v_stride) & 1) && !(page_stride & 1) &&
                                 !(((uintptr_t)k | (uintptr_t)v | (uintptr_t)k_cache | (uintptr_t)v_cache) & 7))) &&
                    (rot == 0 || !((uintptr_t)cos_sin & 7));
  const dim3 grid(rows, shares);
  int rc;
#define STORE_GO(T) \
  rc = even ? launch_pdl(qkv_store_kernel<T, true>, grid, threads, 0, stream, a) \
            : launch_pdl(qkv_store_kernel<T, false>, grid, threads, 0, stream, a)
  if (dtype == LLM_F32) STORE_GO(float);
  else if (dtype == LLM_BF16) STORE_GO(bf16);
  else return LLM_ERR_UNSUPPORTED;
#undef STORE_GO
  return launched_many_blocks(rc, (long long)rows * shares);
}

LLM_EXPORT int llm_qkv_store(const float* q, int q_stride, const float* k, int k_stride, const float* v,
                             int v_stride, const float* q_w, const float* k_w, const float* cos_sin, void* q_out,
                             void* k_cache, void* v_cache, int dtype, long long page_stride, const int* table,
                             int table_stride, const int* row_slot, const int* row_pos, int rows, int Hq, int Hkv,
                             int d, int dv, int hd, int rot, int norm, float eps, int page_size, int has_kv,
                             cudaStream_t stream) {
  return llm_qkv_store_mix(q, q_stride, k, k_stride, v, v_stride, q_w, k_w, cos_sin, q_out, k_cache, v_cache, dtype,
                           page_stride, table, table_stride, row_slot, row_pos, rows, Hq, Hkv, d, dv, hd, rot, norm,
                           eps, page_size, has_kv, 0.f, 0, nullptr, 0, 0.f, stream);
}

LLM_EXPORT int llm_pool_blocks(const void* k_cache, const void* v_cache, long long page_stride, const int* table,
                               int table_stride, void* pk_cache, void* pv_cache, long long p_page_stride,
                               const int* p_table, int p_table_stride, const int* row_slot, const int* row_pos,
                               int dtype, int rows, int Hkv, int hd, int page_size, int P, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (P <= 0 || Hkv <= 0 || Hkv > 65535) return LLM_ERR_ARGUMENT;
  if (hd <= 0 || hd > 1024) return LLM_ERR_UNSUPPORTED;
  const dim3 grid(rows, Hkv);
  int subs = hd >= 256 ? 1 : 256 / hd;
  if (subs > P) subs = P;
  const int threads = (subs * hd + 31) / 32 * 32;
  const int smem = subs * 2 * hd * (int)sizeof(float);
  int rc;
  if (dtype == LLM_F32)
    rc = launch_pdl(pool_blocks_kernel<float>, grid, threads, smem, stream, (const float*)k_cache,
                    (const float*)v_cache, page_stride, table, table_stride, (float*)pk_cache, (float*)pv_cache,
                    p_page_stride, p_table, p_table_stride, row_slot, row_pos, Hkv, hd, page_size, P, subs);
  else if (dtype == LLM_BF16)
    rc = launch_pdl(pool_blocks_kernel<bf16>, grid, threads, smem, stream, (const bf16*)k_cache,
                    (const bf16*)v_cache, page_stride, table, table_stride, (bf16*)pk_cache, (bf16*)pv_cache,
                    p_page_stride, p_table, p_table_stride, row_slot, row_pos, Hkv, hd, page_size, P, subs);
  else return LLM_ERR_UNSUPPORTED;
  return launched_many_blocks(rc, (long long)rows * Hkv);
}
