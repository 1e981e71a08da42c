// Embedding gather, RMS norm, SiLU gating and small bookkeeping kernels.
#include "common.cuh"

int g_llm_pdl = 1;
int g_llm_after_rotation = 0;
int g_llm_next_plain = 0;
LLM_EXPORT void llm_set_pdl(int on) { g_llm_pdl = on ? 1 : 0; }

// x[t][:] = table[token[t]][:] * scale   (residual stream is 32-bit in every mode)
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ x, int width, int vocab, int* __restrict__ err, float scale) {
  // The first kernel of a step's layers waits BEFORE it lets its dependents start: no kernel
  // after it can begin, not even the part before its own wait, until everything ahead of the
  // embedding (the step's token, position and block-table updates) is complete.  Kernels of the
  // layers rely on that when they read block tables and old cache pages before their wait.
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) atomicExch(err, 1 + t);
    for (int i = threadIdx.x; i < width; i += blockDim.x) x[(size_t)t * width + i] = 0.f;
    return;
  }
  const T* row = table + (size_t)tok * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) x[(size_t)t * width + i] = to_f32(row[i]) * scale;
}

LLM_EXPORT int llm_embed_scaled(const int* tokens, const void* table, int table_dtype, float* x, int rows,
                                int width, int vocab, int* err_flag, float scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (table_dtype == LLM_F32)
    return launch_pdl(embed_kernel<float>, rows, threads, 0, stream, tokens, (const float*)table, x, width, vocab,
                      err_flag, scale);
  if (table_dtype == LLM_BF16)
    return launch_pdl(embed_kernel<bf16>, rows, threads, 0, stream, tokens, (const bf16*)table, x, width, vocab,
                      err_flag, scale);
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_embed(const int* tokens, const void* table, int table_dtype, float* x, int rows,
                         int width, int vocab, int* err_flag, cudaStream_t stream) {
  return llm_embed_scaled(tokens, table, table_dtype, x, rows, width, vocab, err_flag, 1.f, stream);
}

// y[r][:] = x[src(r)][:] * rsqrt(mean(x^2) + eps) * w[:]    sums and scale in 32-bit.
// src(r) = rows_index ? rows_index[r] : r.
template <typename TOut>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                TOut* __restrict__ y, const int* __restrict__ rows_index, int width,
                                float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows_index ? rows_index[r] : r) * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = xr[i];
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    y[(size_t)r * width + i] = from_f32<TOut>(xr[i] * scale * w[i]);
}

// The same for widths that are multiples of four and at most 256 * 4 * VEC_MAX: the row is read
// once with 16-byte loads and kept in registers between the sum and the scaling.
constexpr int VEC_MAX = 8;
template <typename TOut>
__global__ void __launch_bounds__(256) rms_norm_vec_kernel(const float* __restrict__ x,
                                                           const float* __restrict__ w, TOut* __restrict__ y,
                                                           const int* __restrict__ rows_index, int width,
                                                           float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows_index ? rows_index[r] : r) * width);
  const float4* wr = reinterpret_cast<const float4*>(w);
  const int n4 = width >> 2;
  float4 v[VEC_MAX];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VEC_MAX; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      v[k] = xr[i];
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
  for (int k = 0; k < VEC_MAX; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      const float4 g = wr[i];
      const float a = v[k].x * scale * g.x, b = v[k].y * scale * g.y, c = v[k].z * scale * g.z,
                  d = v[k].w * scale * g.w;
      TOut* dst = y + (size_t)r * width + 4 * i;
      if (sizeof(TOut) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = packed;
      }
    }
  }
}

// Many rows of a narrow width (at most 32 * 4 * WARP_VEC values): a warp per row, eight rows per
// block, no block-wide barrier.  With a block per row a row of 1,024 values is one 16-byte load
// per thread and two barriers, and the kernel is bound by launching blocks (8.6 us for 2,048
// rows of 1,024 against 3 us here).
constexpr int WARP_VEC = 16;
template <typename TOut>
__global__ void __launch_bounds__(256) rms_norm_warp_kernel(const float* __restrict__ x,
                                                            const float* __restrict__ w, TOut* __restrict__ y,
                                                            const int* __restrict__ rows_index, int rows,
                                                            int width, float eps) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows_index ? rows_index[r] : r) * width);
  const float4* wr = reinterpret_cast<const float4*>(w);
  const int n4 = width >> 2;
  float4 v[WARP_VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < WARP_VEC; ++k) {
    const int i = lane + k * 32;
    if (i < n4) {
      v[k] = xr[i];
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
  for (int k = 0; k < WARP_VEC; ++k) {
    const int i = lane + k * 32;
    if (i < n4) {
      const float4 g = wr[i];
      const float a = v[k].x * scale * g.x, b = v[k].y * scale * g.y, c = v[k].z * scale * g.z,
                  d = v[k].w * scale * g.w;
      TOut* dst = y + (size_t)r * width + 4 * i;
      if (sizeof(TOut) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = packed;
      }
    }
  }
}

LLM_EXPORT int llm_rms_norm(const float* x, const float* w, void* y, int out_dtype,
                            const int* rows_index, int rows, int width, float eps,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  const bool vec = width % 4 == 0 && width <= 256 * 4 * VEC_MAX &&
                   (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0;
  if (vec && rows >= 512 && width <= 32 * 4 * WARP_VEC) {
    const int blocks = (rows + 7) / 8;
    if (out_dtype == LLM_F32)
      return launch_pdl(rms_norm_warp_kernel<float>, blocks, 256, 0, stream, x, w, (float*)y, rows_index, rows,
                        width, eps);
    if (out_dtype == LLM_BF16)
      return launch_pdl(rms_norm_warp_kernel<bf16>, blocks, 256, 0, stream, x, w, (bf16*)y, rows_index, rows,
                        width, eps);
    return LLM_ERR_UNSUPPORTED;
  }
  if (vec) {
    if (out_dtype == LLM_F32)
      return launch_pdl(rms_norm_vec_kernel<float>, rows, 256, 0, stream, x, w, (float*)y, rows_index, width, eps);
    if (out_dtype == LLM_BF16)
      return launch_pdl(rms_norm_vec_kernel<bf16>, rows, 256, 0, stream, x, w, (bf16*)y, rows_index, width, eps);
    return LLM_ERR_UNSUPPORTED;
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  if (out_dtype == LLM_F32)
    return launch_pdl(rms_norm_kernel<float>, rows, threads, 0, stream, x, w, (float*)y, rows_index, width, eps);
  if (out_dtype == LLM_BF16)
    return launch_pdl(rms_norm_kernel<bf16>, rows, threads, 0, stream, x, w, (bf16*)y, rows_index, width, eps);
  return LLM_ERR_UNSUPPORTED;
}

// out[t][j] = silu(gu[t][j]) * gu[t][ff + j]   with silu(z) = z / (1 + exp(-z)), in 32-bit.
template <typename TOut>
__global__ void silu_mul_kernel(const float* __restrict__ gate_up, TOut* __restrict__ out,
                                long long total, int ff) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const long long t = idx / ff;
    const int j = (int)(idx - t * ff);
    const float g = gate_up[t * 2 * ff + j];
    const float u = gate_up[t * 2 * ff + ff + j];
    out[idx] = from_f32<TOut>(g / (1.0f + expf(-g)) * u);
  }
}

LLM_EXPORT int llm_silu_mul(const float* gate_up, void* out, int out_dtype, int rows, int ff,
                            cudaStream_t stream) {
  const long long total = (long long)rows * ff;
  if (total <= 0) return 0;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (out_dtype == LLM_F32)
    silu_mul_kernel<float><<<blocks, threads, 0, stream>>>(gate_up, (float*)out, total, ff);
  else if (out_dtype == LLM_BF16)
    silu_mul_kernel<bf16><<<blocks, threads, 0, stream>>>(gate_up, (bf16*)out, total, ff);
  else
    return LLM_ERR_UNSUPPORTED;
  return launch_status();
}

// out[t][j] += bias[j], in 32-bit, rounded once to the type of out: the bias of a projection
// (the reference adds it after the product, crates/engine/model/src/forward.rs:810-830).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, const float* __restrict__ bias, long long total,
                                int width) {
  pdl_trigger();
  pdl_wait();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) out[idx] = from_f32<T>(to_f32(out[idx]) + bias[idx % width]);
}

LLM_EXPORT int llm_add_bias(void* out, int dtype, const float* bias, int rows, int width,
                            cudaStream_t stream) {
  const long long total = (long long)rows * width;
  if (total <= 0) return 0;
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == LLM_F32)
    return launch_pdl(add_bias_kernel<float>, blocks, threads, 0, stream, (float*)out, bias, total, width);
  if (dtype == LLM_BF16)
    return launch_pdl(add_bias_kernel<bf16>, blocks, threads, 0, stream, (bf16*)out, bias, total, width);
  return LLM_ERR_UNSUPPORTED;
}

// Scatter (row, column, value) triples into a table of block ids kept on the device.
__global__ void table_update_kernel(int* __restrict__ table, int row_stride,
                                    const int* __restrict__ updates, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) table[(size_t)updates[3 * i] * row_stride + updates[3 * i + 1]] = updates[3 * i + 2];
}

// The same with the number of triples read from device memory (at most max_n), so that the
// launch itself does not change from step to step.
__global__ void table_update_counted_kernel(int* __restrict__ table, int row_stride,
                                            const int* __restrict__ updates,
                                            const int* __restrict__ count, int max_n) {
  pdl_trigger();
  pdl_wait();
  const int n = min(*count, max_n);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    table[(size_t)updates[3 * i] * row_stride + updates[3 * i + 1]] = updates[3 * i + 2];
}

LLM_EXPORT int llm_table_update_counted(int* table, int row_stride, const int* updates,
                                        const int* count, int max_n, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  const int blocks = (max_n + 127) / 128 < 8 ? (max_n + 127) / 128 : 8;
  return launch_pdl(table_update_counted_kernel, blocks, 128, 0, stream, table, row_stride, updates, count, max_n);
}

LLM_EXPORT int llm_table_update(int* table, int row_stride, const int* updates, int n,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  table_update_kernel<<<(n + 127) / 128, 128, 0, stream>>>(table, row_stride, updates, n);
  return launch_status();
}

// tokens[i] = source[index[i]] where index[i] >= 0: rows whose token was drawn by the previous
// step and has not been to the host yet take it from the sampler's output on the device.
__global__ void patch_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ source,
                                    const int* __restrict__ index, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && index[i] >= 0) tokens[i] = source[index[i]];
}

LLM_EXPORT int llm_patch_tokens(int* tokens, const int* source, const int* index, int n,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  patch_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, source, index, n);
  return launch_status();
}

// Clear a [rows][cols] float matrix with row stride ld (a kernel rather than a memset, so that it
// can take part in programmatic dependent launch).
__global__ void zero_f32_kernel(float* __restrict__ p, int rows, int cols, int ld) {
  pdl_trigger();
  pdl_wait();
  const long long total = (long long)rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    p[(i / cols) * ld + (i % cols)] = 0.f;
}

int llm_zero_f32(float* p, int rows, int cols, int ld, cudaStream_t stream) {
  const long long total = (long long)rows * cols;
  if (total <= 0) return 0;
  const int blocks = (int)((total + 1023) / 1024 < 592 ? (total + 1023) / 1024 : 592);
  return launch_pdl(zero_f32_kernel, blocks, 256, 0, stream, p, rows, cols, ld);
}

// state[slots[i]][:] = 0 for i < *count (count read on the device, at most max_n): the fixed-size
// state of request slots that were opened for this step, cleared inside the step so that a
// recorded step clears whatever slots its replay names.
__global__ void zero_slots_kernel(unsigned int* __restrict__ state, long long row_words,
                                  const int* __restrict__ slots, const int* __restrict__ count) {
  pdl_wait();
  pdl_trigger();
  if ((int)blockIdx.x >= *count) return;
  unsigned int* row = state + (size_t)slots[blockIdx.x] * row_words;
  for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < row_words;
       i += (long long)gridDim.y * blockDim.x)
    row[i] = 0u;
}

LLM_EXPORT int llm_zero_slots(void* state, long long row_bytes, const int* slots, const int* count,
                              int max_n, cudaStream_t stream) {
  if (max_n <= 0 || row_bytes <= 0) return 0;
  if (row_bytes % 4 != 0 || ((uintptr_t)state & 3)) return LLM_ERR_UNSUPPORTED;
  const long long words = row_bytes / 4;
  const int chunks = (int)((words + 4095) / 4096 < 64 ? (words + 4095) / 4096 : 64);
  return launch_pdl(zero_slots_kernel, dim3(max_n, chunks), 256, 0, stream, (unsigned int*)state, words,
                    slots, count);
}

// A wait that runs out, on purpose and harmlessly: one thread waits on an mbarrier at which
// nothing arrives, with a caller-given limit of clock cycles, gives up, records role 99 in the
// status word and returns.  Every bounded wait of the TMA / tcgen05 kernels ends this way when
// its limit passes; tests use this kernel to see the host side of that path (the status word
// reaching the engine, the step's requests failing) without a kernel that misbehaves.
__global__ void selftest_wait_kernel(int* status, long long limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait(&bar, 0, limit)) atomicExch(status, 99);
  }
}

LLM_EXPORT int llm_selftest_wait_gives_up(int* status, long long limit_cycles, cudaStream_t stream) {
  if (status == nullptr || limit_cycles <= 0 || limit_cycles > 2000000) return LLM_ERR_ARGUMENT;
  selftest_wait_kernel<<<1, 32, 0, stream>>>(status, limit_cycles);
  return launch_status();
}

// out[r][c] = x[r][c] rounded to the output type, for a [rows][cols] window of two matrices with
// their own row strides (the 32-bit residual stream as a sublayer's input; a slice of a
// projection's 32-bit output as the next product's operand).
template <typename TOut>
__global__ void cast_rows_kernel(const float* __restrict__ x, long long x_stride, TOut* __restrict__ out,
                                 long long out_stride, int rows, int cols) {
  pdl_trigger();
  pdl_wait();
  const long long total = (long long)rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols, c = i - r * cols;
    out[r * out_stride + c] = from_f32<TOut>(x[r * x_stride + c]);
  }
}

// The same, four values per thread: rows of whole 16-byte units on both sides.
template <typename TOut>
__global__ void cast_rows_vec_kernel(const float* __restrict__ x, long long x_stride, TOut* __restrict__ out,
                                     long long out_stride, int rows, int cols4) {
  pdl_trigger();
  pdl_wait();
  const long long total = (long long)rows * cols4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols4, c = (i - r * cols4) * 4;
    const float4 v = *reinterpret_cast<const float4*>(x + r * x_stride + c);
    TOut* dst = out + r * out_stride + c;
    if (sizeof(TOut) == 4) {
      *reinterpret_cast<float4*>(dst) = v;
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst) = packed;
    }
  }
}

LLM_EXPORT int llm_cast_rows(const float* x, long long x_stride, void* out, int out_dtype,
                             long long out_stride, int rows, int cols, cudaStream_t stream) {
  const long long total = (long long)rows * cols;
  if (total <= 0) return 0;
  if (cols % 4 == 0 && x_stride % 4 == 0 && out_stride % 4 == 0 &&
      (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
    const long long t4 = total / 4;
    const int vb = (int)((t4 + 255) / 256 < 2368 ? (t4 + 255) / 256 : 2368);
    if (out_dtype == LLM_F32)
      return launch_pdl(cast_rows_vec_kernel<float>, vb, 256, 0, stream, x, x_stride, (float*)out, out_stride, rows, cols / 4);
    if (out_dtype == LLM_BF16)
      return launch_pdl(cast_rows_vec_kernel<bf16>, vb, 256, 0, stream, x, x_stride, (bf16*)out, out_stride, rows, cols / 4);
    return LLM_ERR_UNSUPPORTED;
  }
  const int blocks = (int)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
  if (out_dtype == LLM_F32)
    return launch_pdl(cast_rows_kernel<float>, blocks, 256, 0, stream, x, x_stride, (float*)out, out_stride, rows, cols);
  if (out_dtype == LLM_BF16)
    return launch_pdl(cast_rows_kernel<bf16>, blocks, 256, 0, stream, x, x_stride, (bf16*)out, out_stride, rows, cols);
  return LLM_ERR_UNSUPPORTED;
}

// x[r][:] += y[r][:] * rsqrt(mean(y[r]^2) + eps) * w[:] * s[:]: the norm of a sublayer's output,
// a scale per channel (s may be null), and the residual sum, all in 32-bit.  With `h` the new x
// is also written there rounded to bfloat16: the next sublayer's input, without a pass of its own.
// With `clear` y is left holding zeros (the product that fills it adds partial sums into it).
__global__ void norm_scale_add_kernel(float* __restrict__ y, const float* __restrict__ w,
                                      const float* __restrict__ s, float* __restrict__ x,
                                      bf16* __restrict__ h, int width, float eps, int clear) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t r = blockIdx.x;
  float* yr = y + r * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = yr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = yr[i] * scale * w[i];
    if (clear) yr[i] = 0.f;
    if (s) v *= s[i];
    v += x[r * width + i];
    x[r * width + i] = v;
    if (h) h[r * width + i] = __float2bfloat16_rn(v);
  }
}

// The same for widths that are multiples of four and at most 256 * 4 * VEC_MAX: the row of y is
// read once with 16-byte loads and kept in registers between the sum and the scaling.
__global__ void __launch_bounds__(256) norm_scale_add_vec_kernel(float* __restrict__ y, const float* __restrict__ w,
                                                                 const float* __restrict__ s, float* __restrict__ x,
                                                                 bf16* __restrict__ h, int width, float eps,
                                                                 int clear) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t r = blockIdx.x;
  float4* yr = reinterpret_cast<float4*>(y + r * width);
  float4* xr = reinterpret_cast<float4*>(x + r * width);
  const float4* wr = reinterpret_cast<const float4*>(w);
  const float4* sr = reinterpret_cast<const float4*>(s);
  const int n4 = width >> 2;
  float4 v[VEC_MAX];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VEC_MAX; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      v[k] = yr[i];
      if (clear) yr[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
  for (int k = 0; k < VEC_MAX; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      const float4 g = wr[i], o = xr[i];
      float a = v[k].x * scale * g.x, b = v[k].y * scale * g.y, c = v[k].z * scale * g.z,
            d = v[k].w * scale * g.w;
      if (s) {
        const float4 t = sr[i];
        a *= t.x, b *= t.y, c *= t.z, d *= t.w;
      }
      a += o.x, b += o.y, c += o.z, d += o.w;
      xr[i] = make_float4(a, b, c, d);
      if (h) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(h + r * width + 4 * i) = packed;
      }
    }
  }
}

LLM_EXPORT int llm_norm_scale_add(float* y, const float* w, const float* s, float* x, void* h, int rows,
                                  int width, float eps, int clear, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (width % 4 == 0 && width <= 256 * 4 * VEC_MAX &&
      (((uintptr_t)y | (uintptr_t)w | (uintptr_t)s | (uintptr_t)x | (uintptr_t)h) & 15) == 0)
    return launch_pdl(norm_scale_add_vec_kernel, rows, 256, 0, stream, y, w, s, x, (bf16*)h, width, eps, clear);
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  return launch_pdl(norm_scale_add_kernel, rows, threads, 0, stream, y, w, s, x, (bf16*)h, width, eps, clear);
}

// out[r][h][:] *= sigmoid(gate[r * gate_stride + h]): one gate per (row, head) on the output of
// attention, in 32-bit, rounded once.  With `clear` the gates that were read are zeroed (they
// lie in a buffer that a split-K product adds into).
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, float* __restrict__ gate, int gate_stride, int rows,
                                 int H, int hd, int clear) {
  pdl_trigger();
  pdl_wait();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)rows * H) return;
  const int r = (int)(item / H), h = (int)(item % H), lane = threadIdx.x & 31;
  float* gp = gate + (size_t)r * gate_stride + h;
  const float z = *gp;
  __syncwarp();
  if (clear && lane == 0) *gp = 0.f;
  const float sg = 1.f / (1.f + expf(-z));
  T* o = out + ((size_t)r * H + h) * hd;
  for (int i = lane; i < hd; i += 32) o[i] = from_f32<T>(to_f32(o[i]) * sg);
}

LLM_EXPORT int llm_head_gate(void* out, int dtype, float* gate, int gate_stride, int rows, int H, int hd,
                             int clear, cudaStream_t stream) {
  const long long items = (long long)rows * H;
  if (items <= 0) return 0;
  const int blocks = (int)((items + 3) / 4);
  if (dtype == LLM_F32)
    return launched_many_blocks(launch_pdl(head_gate_kernel<float>, blocks, 128, 0, stream, (float*)out, gate,
                                           gate_stride, rows, H, hd, clear), blocks);
  if (dtype == LLM_BF16)
    return launched_many_blocks(launch_pdl(head_gate_kernel<bf16>, blocks, 128, 0, stream, (bf16*)out, gate,
                                           gate_stride, rows, H, hd, clear), blocks);
  return LLM_ERR_UNSUPPORTED;
}

// out[r][c] *= sigmoid(gate[r * gate_stride + c]): one gate per channel on the output of
// attention, in 32-bit, rounded once.  With `clear` the gates that were read are zeroed.
template <typename T>
__global__ void channel_gate_kernel(T* __restrict__ out, float* __restrict__ gate, int gate_stride, int cols,
                                    long long total, int clear) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    float* gp = gate + r * gate_stride + (i - r * cols);
    const float z = *gp;
    if (clear) *gp = 0.f;
    out[i] = from_f32<T>(to_f32(out[i]) / (1.f + expf(-z)));
  }
}

LLM_EXPORT int llm_channel_gate(void* out, int dtype, float* gate, int gate_stride, int rows, int cols, int clear,
                                cudaStream_t stream) {
  const long long total = (long long)rows * cols;
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 4736 ? (total + 255) / 256 : 4736);
  // (it stands in front of the output projection: see launched_many_blocks)
  if (dtype == LLM_F32)
    return launched_many_blocks(launch_pdl(channel_gate_kernel<float>, blocks, 256, 0, stream, (float*)out, gate,
                                           gate_stride, cols, total, clear), blocks);
  if (dtype == LLM_BF16)
    return launched_many_blocks(launch_pdl(channel_gate_kernel<bf16>, blocks, 256, 0, stream, (bf16*)out, gate,
                                           gate_stride, cols, total, clear), blocks);
  return LLM_ERR_UNSUPPORTED;
}
