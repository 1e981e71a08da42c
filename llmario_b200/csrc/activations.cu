// Small passes behind a product that the standard feed-forward and head do not have: a gated
// activation with a choice of function and an optional bias on both halves, an activation without
// a gate, a scaled soft cap, and the mean of two normed rows (the join of two mixers that run
// side by side).
#include "common.cuh"

namespace {
enum ActKind : int { ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_CLAMPED_SWISH = 2, ACT_RELU_SQUARED = 3 };
constexpr float SWISH_SLOPE = 1.702f;      // of the clamped gate: g * sigmoid(1.702 g)

__device__ __forceinline__ float act_f(float z, int kind) {
  if (kind == ACT_GELU_TANH)     // 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.f + expf(-z));
}

// out[t][j] = act(gu[t][j] + b[j]) * (gu[t][ff + j] + b[ff + j]), in 32-bit, rounded once.
// clear: what was read of gu is zeroed (it lies in a buffer that a split-K product adds into).
template <typename TOut>
__global__ void gated_act_kernel(float* __restrict__ gate_up, const float* __restrict__ bias,
                                 TOut* __restrict__ out, long long total, int ff, int kind, int clear,
                                 float limit) {
  pdl_trigger();
  pdl_wait();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const long long t = idx / ff;
    const int j = (int)(idx - t * ff);
    float g = gate_up[t * 2 * ff + j], u = gate_up[t * 2 * ff + ff + j];
    if (clear) gate_up[t * 2 * ff + j] = 0.f, gate_up[t * 2 * ff + ff + j] = 0.f;
    if (bias) g += bias[j], u += bias[ff + j];
    if (kind == ACT_CLAMPED_SWISH) {
      // the gate bounded above, the other half on both sides, and one added to it
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      out[idx] = from_f32<TOut>(g / (1.f + expf(-SWISH_SLOPE * g)) * (u + 1.f));
    } else {
      out[idx] = from_f32<TOut>(act_f(g, kind) * u);
    }
  }
}

// out[t][j] = act(x[t][j]) for an activation without a gate (the square of relu), rounded once
template <typename TOut>
__global__ void act_rows_kernel(float* __restrict__ x, TOut* __restrict__ out, long long total, int kind,
                                int clear) {
  pdl_trigger();
  pdl_wait();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const float v = fmaxf(x[idx], 0.f);
    if (clear) x[idx] = 0.f;
    out[idx] = from_f32<TOut>(v * v);
  }
}

// y[r] (+)= (unit(a[r]) * wa + unit(b[r]) * wb) / 2, unit(.) = a row over its root mean square (eps
// inside the root); one block per row, all 32-bit
__global__ void __launch_bounds__(256) dual_norm_mean_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                             const float* __restrict__ wa,
                                                             const float* __restrict__ wb, float* __restrict__ y,
                                                             int width, float eps, int accumulate) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * width;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    sa = fmaf(a[row + c], a[row + c], sa);
    sb = fmaf(b[row + c], b[row + c], sb);
  }
  const float ra = rsqrtf(block_sum(sa, scratch) / (float)width + eps);
  const float rb = rsqrtf(block_sum(sb, scratch) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = 0.5f * (a[row + c] * ra * wa[c] + b[row + c] * rb * wb[c]);
    y[row + c] = accumulate ? y[row + c] + v : v;
  }
}

// z <- cap * tanh(z * scale / cap)   (cap <= 0: z <- z * scale)
__global__ void scale_soft_cap_kernel(float* __restrict__ z, long long total, float scale, float cap) {
  pdl_trigger();
  pdl_wait();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const float v = z[idx] * scale;
    z[idx] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}
}  // namespace

// (limit: the bound of the clamped form, unused by the others)
LLM_EXPORT int llm_gated_act_limit(float* gate_up, const float* bias, void* out, int out_dtype, int rows,
                                   int ff, int kind, int clear, float limit, cudaStream_t stream) {
  const long long total = (long long)rows * ff;
  if (total <= 0) return 0;
  if (kind != ACT_SILU && kind != ACT_GELU_TANH && kind != ACT_CLAMPED_SWISH) return LLM_ERR_ARGUMENT;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  if (out_dtype == LLM_F32)
    return launched_many_blocks(
        launch_pdl(gated_act_kernel<float>, blocks, 256, 0, stream, gate_up, bias, (float*)out, total, ff, kind, clear, limit), blocks);
  if (out_dtype == LLM_BF16)
    return launched_many_blocks(
        launch_pdl(gated_act_kernel<bf16>, blocks, 256, 0, stream, gate_up, bias, (bf16*)out, total, ff, kind, clear, limit), blocks);
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_gated_act(float* gate_up, const float* bias, void* out, int out_dtype, int rows,
                             int ff, int kind, int clear, cudaStream_t stream) {
  if (kind == ACT_CLAMPED_SWISH) return LLM_ERR_ARGUMENT;
  return llm_gated_act_limit(gate_up, bias, out, out_dtype, rows, ff, kind, clear, 0.f, stream);
}

LLM_EXPORT int llm_act_rows(float* x, void* out, int out_dtype, long long total, int kind, int clear,
                            cudaStream_t stream) {
  if (total <= 0) return 0;
  if (kind != ACT_RELU_SQUARED) return LLM_ERR_ARGUMENT;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  if (out_dtype == LLM_F32)
    return launched_many_blocks(launch_pdl(act_rows_kernel<float>, blocks, 256, 0, stream, x, (float*)out, total,
                                           kind, clear), blocks);
  if (out_dtype == LLM_BF16)
    return launched_many_blocks(launch_pdl(act_rows_kernel<bf16>, blocks, 256, 0, stream, x, (bf16*)out, total,
                                           kind, clear), blocks);
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_dual_norm_mean(const float* a, const float* b, const float* wa, const float* wb, float* y,
                                  int rows, int width, float eps, int accumulate, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  return launched_many_blocks(
      launch_pdl(dual_norm_mean_kernel, rows, 256, 0, stream, a, b, wa, wb, y, width, eps, accumulate), rows);
}

LLM_EXPORT int llm_scale_soft_cap(float* z, long long total, float scale, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  return launch_pdl(scale_soft_cap_kernel, blocks, 256, 0, stream, z, total, scale, cap);
}
