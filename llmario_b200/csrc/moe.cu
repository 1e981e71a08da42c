// A feed-forward of routed experts.  Per token the router's logits choose `top` of E small gated
// feed-forwards; their outputs are summed with the softmax of the chosen logits as weights.
//   route:    ids[r][k], wts[r][k]  from  z[r][0:E]                      (32-bit)
//   gate/up:  act[r][k][f] = silu(Wg_e[f] . h_r) * (Wu_e[f] . h_r),  e = ids[r][k]
//   down:     y[r][c] (+)= sum_k wts[r][k] * (Wd_e[c] . act[r][k])  [+ sigmoid(g_r) * shared[r][c]]
// The row-wise kernels here give every (token, chosen expert) its own matrix-vector products:
// the form for steps of few rows, where a token's experts are read once each and nothing has
// to be sorted; which expert a row uses is read on the device, so recorded steps replay.
// Sums run in a fixed order per output, so a row's result does not depend on the batch.
//
// The grouped form, for 16-bit models on the tensor cores: the (token, chosen expert) pairs are
// sorted by expert into a padded buffer in which every expert's rows start a tile of `bn` rows
// (align), the tokens' inputs are copied there (gather), two grouped products
// (llm_gemm_tcgen05_grouped: each tile of rows with its expert's matrices) make the gated
// activation and the experts' outputs, and one pass sums a token's outputs with its weights
// (combine).  Every expert in use is read once per tile of its rows, whatever the step's size;
// all of it is decided on the device, so recorded steps replay.
#include "common.cuh"

namespace {
constexpr int MAX_TOP = 16;

// The choice of one row by one warp, from its E router outputs zr (shared or global memory).
// mode 0: the k-th choice is the largest logit not chosen before (the lowest index among equals);
// the weights are a softmax in which only the chosen logits take part.  mode 1: scores are the
// softmax over all E outputs; the choice goes by score + corr[e] (the same tie rule), the weight
// of a chosen expert is its score, not renormalised.  mode 2: as mode 1, but the weights are the
// chosen scores over their sum (+ 1e-20), times `wscale`.
__device__ __forceinline__ void choose_row(const float* zr, int E, int top, int mode, const float* __restrict__ corr,
                                           int lane, int* __restrict__ ids, float* __restrict__ wts,
                                           float wscale = 1.f) {
  const bool renorm = mode == 2;
  if (renorm) mode = 1;
  float zmax = 0.f, inv_sum = 1.f;
  if (mode == 1) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
    zmax = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(zr[e] - zmax);
    inv_sum = 1.f / warp_sum(sum);
  }
  float best[MAX_TOP];
  int pick[MAX_TOP];
  for (int k = 0; k < top; ++k) {
    float v = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= pick[j] == e;
      const float x = mode == 1 ? expf(zr[e] - zmax) * inv_sum + (corr ? corr[e] : 0.f) : zr[e];
      if (!taken && (x > v || (x == v && e < at) || at == 0x7fffffff)) v = x, at = e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (oa != 0x7fffffff && (at == 0x7fffffff || ov > v || (ov == v && oa < at))) v = ov, at = oa;
    }
    best[k] = v, pick[k] = at;
  }
  if (lane == 0) {
    if (mode == 1) {
      float chosen = 0.f;
      for (int k = 0; k < top; ++k) {
        ids[k] = pick[k];
        wts[k] = expf(zr[pick[k]] - zmax) * inv_sum;
        chosen += wts[k];
      }
      if (renorm) {
        const float f = wscale / (chosen + 1e-20f);
        for (int k = 0; k < top; ++k) wts[k] *= f;
      }
      return;
    }
    float sum = 0.f;       // best[0] is the largest
    for (int k = 0; k < top; ++k) sum += expf(best[k] - best[0]);
    for (int k = 0; k < top; ++k) {
      ids[k] = pick[k];
      wts[k] = expf(best[k] - best[0]) / sum;
    }
  }
}

// One warp per row.
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ z, int z_stride, int rows, int E,
                                                        int top, int mode, const float* __restrict__ corr,
                                                        int* __restrict__ ids, float* __restrict__ wts,
                                                        float wscale) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  choose_row(z + (size_t)r * z_stride, E, top, mode, corr, lane, ids + (size_t)r * top, wts + (size_t)r * top,
             wscale);
}


// Router logits and the choice in one kernel.  A block takes R rows: their h is staged in shared
// memory in 32-bit, every warp makes, for its experts, the logits z[e] = w[e] . h + b[e] of all R
// rows from one reading of w[e] (w and b 32-bit, sums in a fixed order that does not depend on
// R), then warp i chooses for row i as moe_route_kernel does.  Rows of w behind the E experts'
// (n_out - E of them: the gate of a shared expert) get their logits too; all go to z_out.
template <typename T, int R>
__global__ void __launch_bounds__(256) moe_router_kernel(const T* __restrict__ h, const float* __restrict__ w,
                                                         const float* __restrict__ b, float* __restrict__ z_out,
                                                         int z_stride, int rows, int width, int E, int n_out,
                                                         int top, int mode, const float* __restrict__ corr,
                                                         int* __restrict__ ids, float* __restrict__ wts,
                                                         float wscale) {
  extern __shared__ float rs[];        // h[R][width], z[R][n_out]
  float* h_s = rs;
  float* z_s = rs + (size_t)R * width;
  pdl_trigger();
  pdl_wait();
  const int r0 = blockIdx.x * R, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < R * width; i += blockDim.x) {
    const int rr = i / width, c = i - rr * width;
    h_s[i] = r0 + rr < rows ? to_f32(h[(size_t)(r0 + rr) * width + c]) : 0.f;
  }
  __syncthreads();
  const bool wide = (width & 3) == 0 && ((uintptr_t)w & 15) == 0;
  for (int e = warp; e < n_out; e += nwarps) {
    const float* we = w + (size_t)e * width;
    float acc[R];
#pragma unroll
    for (int rr = 0; rr < R; ++rr) acc[rr] = 0.f;
    if (wide) {
#pragma unroll 4
      for (int i = lane * 4; i < width; i += 128) {
        const float4 a = *reinterpret_cast<const float4*>(we + i);
#pragma unroll
        for (int rr = 0; rr < R; ++rr) {
          const float* hr = h_s + (size_t)rr * width + i;
          acc[rr] = fmaf(a.x, hr[0], acc[rr]), acc[rr] = fmaf(a.y, hr[1], acc[rr]);
          acc[rr] = fmaf(a.z, hr[2], acc[rr]), acc[rr] = fmaf(a.w, hr[3], acc[rr]);
        }
      }
    } else {
      for (int i = lane; i < width; i += 32) {
        const float a = we[i];
#pragma unroll
        for (int rr = 0; rr < R; ++rr) acc[rr] = fmaf(a, h_s[(size_t)rr * width + i], acc[rr]);
      }
    }
#pragma unroll
    for (int rr = 0; rr < R; ++rr) {
      const float sum = warp_sum(acc[rr]);
      if (lane == 0 && r0 + rr < rows) {
        const float v = sum + (b ? b[e] : 0.f);
        z_s[rr * n_out + e] = v;
        z_out[(size_t)(r0 + rr) * z_stride + e] = v;
      }
    }
  }
  __syncthreads();
  if (warp >= R || r0 + warp >= rows) return;
  const int r = r0 + warp;
  choose_row(z_s + warp * n_out, E, top, mode, corr, lane, ids + (size_t)r * top, wts + (size_t)r * top, wscale);
}

template <typename T> __device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ x,
                                                               int n, int lane);
template <> __device__ __forceinline__ float dot_row<float>(const float* __restrict__ w, const float* __restrict__ x,
                                                            int n, int lane) {
  float acc = 0.f;
  for (int i = lane; i < n; i += 32) acc = fmaf(w[i], x[i], acc);
  return warp_sum(acc);
}
template <> __device__ __forceinline__ float dot_row<bf16>(const bf16* __restrict__ w, const float* __restrict__ x,
                                                           int n, int lane) {
  float acc = 0.f;
  if ((n & 7) == 0 && ((uintptr_t)w & 15) == 0) {
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(w + i);
      const uint32_t u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc = fmaf(__uint_as_float(u[j] << 16), x[i + 2 * j], acc);
        acc = fmaf(__uint_as_float(u[j] & 0xffff0000u), x[i + 2 * j + 1], acc);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) acc = fmaf(__bfloat162float(w[i]), x[i], acc);
  }
  return warp_sum(acc);
}

// grid (rows * top, ff tiles of 8); a block stages its row of h in shared memory, a warp makes
// two features.  gate_up: [E][2 ff][width], gate rows first; kind 3 (an expert without a gate,
// act = max(W_up h, 0)^2): [E][ff][width].
template <typename T>
__global__ void __launch_bounds__(128) moe_gate_up_rows_kernel(const T* __restrict__ h, const T* __restrict__ gate_up,
                                                               const int* __restrict__ ids, T* __restrict__ act,
                                                               int width, int ff, int top, int E, int kind,
                                                               float limit) {
  extern __shared__ float h_s[];
  pdl_trigger();
  pdl_wait();
  const int item = blockIdx.x, r = item / top;
  const int e = ids[item];
  if (e < 0 || e >= E) return;       // an identity expert: it has no matrices
  for (int i = threadIdx.x; i < width; i += blockDim.x) h_s[i] = to_f32(h[(size_t)r * width + i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* we = gate_up + (size_t)e * (kind == 3 ? 1 : 2) * ff * width;
  for (int f = blockIdx.y * 8 + warp; f < min(ff, blockIdx.y * 8 + 8); f += 4) {
    const float g = dot_row<T>(we + (size_t)f * width, h_s, width, lane);
    if (kind == 3) {
      const float p = fmaxf(g, 0.f);
      if (lane == 0) act[(size_t)item * ff + f] = from_f32<T>(p * p);
      continue;
    }
    const float u = dot_row<T>(we + (size_t)(ff + f) * width, h_s, width, lane);
    if (lane == 0) {
      float y;
      if (kind == 2) {       // the gate bounded above, the other half on both sides and one added to it
        const float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
        y = gc / (1.f + expf(-1.702f * gc)) * (uc + 1.f);
      } else {
        y = g / (1.f + expf(-g)) * u;
      }
      act[(size_t)item * ff + f] = from_f32<T>(y);
    }
  }
}

// grid (rows, width tiles of 8); a block stages its row's `top` activation vectors, a warp makes two
// output channels.  down: [E][width][ff].
template <typename T>
__global__ void __launch_bounds__(128) moe_down_rows_kernel(const T* __restrict__ act, const T* __restrict__ down,
                                                            const int* __restrict__ ids, const float* __restrict__ wts,
                                                            float* __restrict__ shared, const float* __restrict__ gate,
                                                            int gate_stride, float* __restrict__ y, int width, int ff,
                                                            int top, int accumulate, int clear_shared, int E,
                                                            const T* __restrict__ h) {
  extern __shared__ float a_s[];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  for (int i = threadIdx.x; i < top * ff; i += blockDim.x) {
    const int e = ids[(size_t)r * top + i / ff];
    a_s[i] = e >= 0 && e < E ? to_f32(act[(size_t)r * top * ff + i]) : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = blockIdx.y * 8 + warp; c < min(width, blockIdx.y * 8 + 8); c += 4) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = ids[(size_t)r * top + k];
      // an expert behind the E with matrices is the identity: its output is the input itself
      const float d = e >= 0 && e < E ? dot_row<T>(down + ((size_t)e * width + c) * ff, a_s + (size_t)k * ff, ff, lane)
                                      : to_f32(h[(size_t)r * width + c]);
      sum = fmaf(wts[(size_t)r * top + k], d, sum);
    }
    if (lane == 0) {
      if (shared) {
        sum = fmaf(1.f / (1.f + expf(-gate[(size_t)r * gate_stride])), shared[(size_t)r * width + c], sum);
        if (clear_shared) shared[(size_t)r * width + c] = 0.f;
      }
      float* dst = y + (size_t)r * width + c;
      *dst = accumulate ? *dst + sum : sum;
    }
  }
}
// One block.  pos[i]: the row of pair i (token i / top, choice i % top) in the padded buffer;
// tile_group[t]: the expert of tile t of that buffer, -1 for a tile without rows.  Which row of
// its expert's range a pair gets depends on the order in which threads arrive; the result of a
// row does not depend on where it stands.
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* __restrict__ ids, int n_pairs, int E, int bn,
                                                         int n_tiles, int* __restrict__ pos,
                                                         int* __restrict__ tile_group) {
  extern __shared__ int sh[];       // counts[E], offsets[E], cursor[E]
  int *counts = sh, *offsets = sh + E, *cursor = sh + 2 * E;
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0, cursor[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tile = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = tile * bn;
      const int tiles = (counts[e] + bn - 1) / bn;
      for (int t = 0; t < tiles && tile < n_tiles; ++t) tile_group[tile++] = e;
    }
    for (; tile < n_tiles; ++tile) tile_group[tile] = -1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    pos[i] = (e >= 0 && e < E) ? offsets[e] + atomicAdd(&cursor[e], 1) : 0;
  }
}

// xp[pos[i]][:] = h[i / top][:]
template <typename T>
__global__ void __launch_bounds__(128) moe_gather_kernel(const T* __restrict__ h, const int* __restrict__ pos,
                                                         T* __restrict__ xp, int width, int top,
                                                         const int* __restrict__ ids, int E) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  if (ids && (ids[i] < 0 || ids[i] >= E)) return;      // an identity expert has no row in the buffer
  const T* src = h + (size_t)(i / top) * width;
  T* dst = xp + (size_t)pos[i] * width;
  if ((width * sizeof(T)) % 16 == 0 && (((uintptr_t)h | (uintptr_t)xp) & 15) == 0) {
    const int n = width * sizeof(T) / 16;
    for (int j = threadIdx.x; j < n; j += blockDim.x)
      reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<const uint4*>(src)[j];
  } else {
    for (int j = threadIdx.x; j < width; j += blockDim.x) dst[j] = src[j];
  }
}

// y[r][c] (+)= sum_k wts[r][k] * d[pos[r * top + k]][c]  (+ sigmoid(gate[r]) * shared[r][c]), k ascending
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ d, const int* __restrict__ pos,
                                                          const float* __restrict__ wts,
                                                          float* __restrict__ shared,
                                                          const float* __restrict__ gate, int gate_stride,
                                                          float* __restrict__ y, int width, int top, int accumulate,
                                                          int clear_shared, const int* __restrict__ ids, int E,
                                                          const void* __restrict__ x_id, int x_dtype, int x_stride) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float g = shared ? 1.f / (1.f + expf(-gate[(size_t)r * gate_stride])) : 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      // (with ids: an expert behind the E with matrices is the identity, its output the row of x_id)
      const bool identity = ids && (ids[(size_t)r * top + k] < 0 || ids[(size_t)r * top + k] >= E);
      const float v = !identity ? d[(size_t)pos[(size_t)r * top + k] * width + c]
                      : x_dtype == LLM_BF16 ? to_f32(((const bf16*)x_id)[(size_t)r * x_stride + c])
                                            : ((const float*)x_id)[(size_t)r * x_stride + c];
      sum = fmaf(wts[(size_t)r * top + k], v, sum);
    }
    if (shared) {
      sum = fmaf(g, shared[(size_t)r * width + c], sum);
      if (clear_shared) shared[(size_t)r * width + c] = 0.f;
    }
    float* dst = y + (size_t)r * width + c;
    *dst = accumulate ? *dst + sum : sum;
  }
}
}  // namespace

LLM_EXPORT int llm_moe_align(const int* ids, int n_pairs, int E, int bn, int n_tiles, int* pos, int* tile_group,
                             cudaStream_t stream) {
  if (n_pairs <= 0 || n_tiles <= 0) return 0;
  if (E <= 0 || E > 4096 || bn <= 0) return LLM_ERR_UNSUPPORTED;
  return launch_pdl(moe_align_kernel, 1, 1024, (size_t)3 * E * sizeof(int), stream, ids, n_pairs, E, bn, n_tiles,
                    pos, tile_group);
}

// (ids with E: pairs whose expert is not one of the E with matrices are left out)
LLM_EXPORT int llm_moe_gather(const void* h, const int* pos, void* xp, int dtype, int n_pairs, int width, int top,
                              const int* ids, int E, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (dtype == LLM_F32)
    return launch_pdl(moe_gather_kernel<float>, n_pairs, 128, 0, stream, (const float*)h, pos, (float*)xp, width, top,
                      ids, E);
  if (dtype == LLM_BF16)
    return launch_pdl(moe_gather_kernel<bf16>, n_pairs, 128, 0, stream, (const bf16*)h, pos, (bf16*)xp, width, top,
                      ids, E);
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_moe_combine(const float* d, const int* pos, const float* wts, float* shared,
                               const float* gate, int gate_stride, float* y, int rows, int width, int top,
                               int accumulate, int clear_shared, const int* ids, int E, const void* x_id,
                               int x_dtype, int x_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((shared && !gate) || (ids && !x_id)) return LLM_ERR_ARGUMENT;
  return launched_many_blocks(launch_pdl(moe_combine_kernel, rows, 256, 0, stream, d, pos, wts, shared, gate,
                                         gate_stride, y, width, top, accumulate, clear_shared, ids, E, x_id,
                                         x_dtype, x_stride), rows);
}

// The router: z_out[r][0:n_out] = w h_r + b (w float32 [n_out][width], the first E rows the
// experts'), ids / wts the `top` chosen experts of every row and their weights.
// mode and corr: see choose_row.
// mode, corr and wscale: see choose_row.
LLM_EXPORT int llm_moe_router_scaled(const void* h, int dtype, const float* w, const float* b, float* z_out,
                                     int z_stride, int rows, int width, int E, int n_out, int top, int mode,
                                     const float* corr, int* ids, float* wts, float wscale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (top < 1 || top > MAX_TOP || top > E || n_out < E || mode < 0 || mode > 2) return LLM_ERR_UNSUPPORTED;
  if ((size_t)(width + n_out) * 4 > 200 * 1024) return LLM_ERR_UNSUPPORTED;
  // many rows: four to a block, so that a block reads the router's rows once for four tokens
  const bool four = rows >= 256 && (size_t)4 * (width + n_out) * 4 <= 200 * 1024;
  const int R = four ? 4 : 1;
  const size_t smem = (size_t)R * (width + n_out) * 4;
  const int blocks = (rows + R - 1) / R;
#define ROUTER(T, RR)                                                                                          \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(moe_router_kernel<T, RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    return launch_pdl(moe_router_kernel<T, RR>, blocks, 256, smem, stream, (const T*)h, w, b, z_out, z_stride, \
                      rows, width, E, n_out, top, mode, corr, ids, wts, wscale);                               \
  } while (0)
  if (dtype == LLM_F32) {
    if (four) ROUTER(float, 4);
    ROUTER(float, 1);
  }
  if (dtype == LLM_BF16) {
    if (four) ROUTER(bf16, 4);
    ROUTER(bf16, 1);
  }
#undef ROUTER
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_moe_router(const void* h, int dtype, const float* w, const float* b, float* z_out, int z_stride,
                              int rows, int width, int E, int n_out, int top, int mode, const float* corr,
                              int* ids, float* wts, cudaStream_t stream) {
  return llm_moe_router_scaled(h, dtype, w, b, z_out, z_stride, rows, width, E, n_out, top, mode, corr, ids, wts,
                               1.f, stream);
}

LLM_EXPORT int llm_moe_route_scaled(const float* z, int z_stride, int rows, int E, int top, int mode,
                                    const float* corr, int* ids, float* wts, float wscale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (top < 1 || top > MAX_TOP || top > E || mode < 0 || mode > 2) return LLM_ERR_UNSUPPORTED;
  return launch_pdl(moe_route_kernel, (rows + 3) / 4, 128, 0, stream, z, z_stride, rows, E, top, mode, corr, ids,
                    wts, wscale);
}

LLM_EXPORT int llm_moe_route(const float* z, int z_stride, int rows, int E, int top, int mode, const float* corr,
                             int* ids, float* wts, cudaStream_t stream) {
  return llm_moe_route_scaled(z, z_stride, rows, E, top, mode, corr, ids, wts, 1.f, stream);
}

// E: experts with matrices (a pair whose expert is not one of them is left out); kind 0: silu(g) u,
// 2: the clamped form with `limit` (see activations.cu), 3: no gate, max(u, 0)^2 with gate_up [E][ff][width]
LLM_EXPORT int llm_moe_gate_up_rows(const void* h, const void* gate_up, const int* ids, void* act, int dtype,
                                    int rows, int width, int ff, int top, int E, int kind, float limit,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((ff + 7) / 8 > 65535 || (size_t)width * 4 > 200 * 1024) return LLM_ERR_UNSUPPORTED;
  const dim3 grid(rows * top, (ff + 7) / 8);
  const size_t smem = (size_t)width * 4;
  if (dtype == LLM_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_gate_up_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_pdl(moe_gate_up_rows_kernel<float>, grid, 128, smem, stream, (const float*)h,
                      (const float*)gate_up, ids, (float*)act, width, ff, top, E, kind, limit);
  }
  if (dtype == LLM_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_gate_up_rows_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_pdl(moe_gate_up_rows_kernel<bf16>, grid, 128, smem, stream, (const bf16*)h, (const bf16*)gate_up,
                      ids, (bf16*)act, width, ff, top, E, kind, limit);
  }
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_moe_down_rows(const void* act, const void* down, const int* ids, const float* wts,
                                 float* shared, const float* gate, int gate_stride, float* y, int dtype,
                                 int rows, int width, int ff, int top, int accumulate, int clear_shared,
                                 int E, const void* h, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)top * ff * 4;
  if ((width + 7) / 8 > 65535 || smem > 200 * 1024) return LLM_ERR_UNSUPPORTED;
  if (shared && !gate) return LLM_ERR_ARGUMENT;
  const dim3 grid(rows, (width + 7) / 8);
  if (dtype == LLM_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_down_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_pdl(moe_down_rows_kernel<float>, grid, 128, smem, stream, (const float*)act, (const float*)down,
                      ids, wts, shared, gate, gate_stride, y, width, ff, top, accumulate, clear_shared, E,
                      (const float*)h);
  }
  if (dtype == LLM_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_down_rows_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_pdl(moe_down_rows_kernel<bf16>, grid, 128, smem, stream, (const bf16*)act, (const bf16*)down, ids,
                      wts, shared, gate, gate_stride, y, width, ff, top, accumulate, clear_shared, E, (const bf16*)h);
  }
  return LLM_ERR_UNSUPPORTED;
}
