// Bandwidth-bound kernels around the matrix products: embedding rows, RMSNorm (plain, and
// fused with the sum of split partial products into the residual), SwiGLU, and the step from
// one decode step to the next on the device. One file for float32 and bfloat16 activations;
// sums, norms and the residual are float32 in both.
//
// Formulas as the reference computes them (paths within the reference project):
//   RMSNorm   src/infer/mormot.ai.infer.backend.cpu.pas:1769-1795, tools/cuda/ops.cu:116-150
//   SwiGLU    src/infer/mormot.ai.infer.backend.cpu.pas:1827-1833, tools/cuda/ops.cu:155-178
#include "common.cuh"

MB_DEFINE_LAST_ERROR

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ x, int H, int V, float scale, int copies,
                             size_t copy_stride) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;  // the host refuses such ids before the step
  const TW* row = table + (size_t)id * H;
  float* out = x + (size_t)t * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = to_f32<TW>(row[c]) * scale;  // times 1 is exact
    for (int k = 0; k < copies; ++k) out[k * copy_stride + c] = v;
  }
}

// x[k][t, :] = table[ids[t], :] * scale for each of `copies` residual streams (copy k starts
// copy_stride floats after copy k - 1).
MB_EXPORT int mb_embed(const void* table, int table_dtype, const int* ids, float* x, int T,
                       int H, int V, float scale, int copies, long long copy_stride,
                       void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == MB_F32)
    mb_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)table, ids, x, H, V, scale,
              copies, (size_t)copy_stride);
  else
    mb_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s, (const __nv_bfloat16*)table, ids, x, H, V,
              scale, copies, (size_t)copy_stride);
  MB_CHECK_LAUNCH("mb_embed");
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row. Before the norm, `parts` partial products [parts][T][H] (float32,
// the split-K results of the product before) are added to the residual row in place, in the
// order of the splits: x += p0 + p1 + ...; then y = w * (x * inv).
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ partial,
                               int parts, size_t part_stride, const TW* __restrict__ w,
                               float eps, TO* __restrict__ y, const int* __restrict__ rows,
                               int H) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ float red[33];
  extern __shared__ float rowbuf[];  // H floats when parts > 0
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * H;
  float sum = 0.f;
  if (parts > 0) {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float v = xr[c];
      for (int p = 0; p < parts; ++p) v += partial[p * part_stride + (size_t)src * H + c];
      xr[c] = v;
      rowbuf[c] = v;
      sum = fmaf(v, v, sum);
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float v = xr[c];
      sum = fmaf(v, v, sum);
    }
  }
  sum = block_sum(sum, red);
  if (y == nullptr) return;
  const float inv = 1.0f / sqrtf(sum / (float)H + eps);
  TO* yr = y + (size_t)r * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = parts > 0 ? rowbuf[c] : xr[c];
    const float n = v * inv;  // rounded to float32 before the weight, as the reference does
    yr[c] = from_f32<TO>(to_f32<TW>(w[c]) * n);
  }
}


// The same for rows of 4 * RMS_THREADS * VEC values at most (a multiple of 4): the row is read
// once with 16-byte loads, kept in registers, and written with 8- or 16-byte stores.
template <typename TO, int VEC, int RMS_THREADS, bool PARTIAL>
__global__ void __launch_bounds__(RMS_THREADS)
rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ partial, int parts,
                   size_t part_stride, const void* __restrict__ w, int w_bf16, float eps,
                   TO* __restrict__ y, const int* __restrict__ rows, int H) {
  MB_TRACE_BEGIN();
  __shared__ float red[33];
  const int r = blockIdx.x;
  // Before the wait for the kernel before: what does not depend on it. The row index and the
  // norm's weights were settled by kernels further back (complete once this kernel runs: every
  // kernel of the stream waits for the one before it ahead of letting its successor start).
  // With PARTIAL the kernel before is the matrix product that left its split sums, which
  // wrote nothing else: the residual row itself can be asked for before the wait too, and
  // only the split sums come after it.
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * H;
  float wv[VEC][4];
  if (y != nullptr) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RMS_THREADS + threadIdx.x) * 4;
      if (c >= H) continue;
      if (w_bf16) {  // four weights with one load (c is a multiple of 4)
        const uint2 raw = *(const uint2*)((const __nv_bfloat16*)w + c);
        const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x);
        const float2 hi = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
        wv[i][0] = lo.x; wv[i][1] = lo.y; wv[i][2] = hi.x; wv[i][3] = hi.y;
      } else {
        const float4 raw = *(const float4*)((const float*)w + c);
        wv[i][0] = raw.x; wv[i][1] = raw.y; wv[i][2] = raw.z; wv[i][3] = raw.w;
      }
    }
  }
  float4 v[VEC];
  float sum = 0.f;
  if (PARTIAL) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RMS_THREADS + threadIdx.x) * 4;
      v[i] = c < H ? *(const float4*)(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  mb_grid_wait();
  mb_grid_launch_next();
  if (!PARTIAL) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RMS_THREADS + threadIdx.x) * 4;
      v[i] = c < H ? *(const float4*)(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  if (PARTIAL) {  // a kernel of its own: the loads in flight below cost registers
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RMS_THREADS + threadIdx.x) * 4;
      if (c >= H) continue;
      const float* pp = partial + (size_t)src * H + c;
      // up to eight loads in flight at once, then added in split order
      for (int p0 = 0; p0 < parts; p0 += 8) {
        float4 a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (p0 + j < parts) a[j] = __ldg((const float4*)(pp + (size_t)(p0 + j) * part_stride));
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (p0 + j < parts) {
            v[i].x += a[j].x; v[i].y += a[j].y; v[i].z += a[j].z; v[i].w += a[j].w;
          }
      }
      *(float4*)(xr + c) = v[i];
    }
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i)
    sum = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, sum))));
  sum = block_sum(sum, red);
  if (y == nullptr) return;
  const float inv = 1.0f / sqrtf(sum / (float)H + eps);
  TO* yr = y + (size_t)r * H;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * RMS_THREADS + threadIdx.x) * 4;
    if (c >= H) continue;
    float o[4];
    o[0] = wv[i][0] * (v[i].x * inv);
    o[1] = wv[i][1] * (v[i].y * inv);
    o[2] = wv[i][2] * (v[i].z * inv);
    o[3] = wv[i][3] * (v[i].w * inv);
    if (sizeof(TO) == 4) {
      *(float4*)((float*)yr + c) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
      __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
      *(uint2*)((__nv_bfloat16*)yr + c) = *(uint2*)h;
    }
  }
  MB_TRACE_END(2);
}

template <typename TW, typename TO>
static int rmsnorm_launch(float* x, const float* partial, int parts, size_t part_stride,
                          const void* w, float eps, void* y, const int* rows, int R, int H,
                          cudaStream_t s) {
  const bool aligned = ((uintptr_t)x & 15) == 0 && ((uintptr_t)partial & 15) == 0 &&
                       (part_stride & 3) == 0 && ((uintptr_t)y & 15) == 0;
  if (H % 4 == 0 && H <= 4 * 1024 * 4 && aligned && ((uintptr_t)w & 15) == 0) {
    // few rows (a decode step) or wide rows: 1024 threads a row, so that a thread waits for few
    // loads; many rows: 256 threads a row and more rows per SM
    const int w_bf16 = sizeof(TW) == 2;
#define RMS_GO(V_, T_)                                                                      \
  if (parts > 0)                                                                            \
    mb_launch(rmsnorm_vec_kernel<TO, V_, T_, true>, dim3(R), dim3(T_), 0, s, x, partial,    \
              parts, part_stride, w, w_bf16, eps, (TO*)y, rows, H);                         \
  else                                                                                      \
    mb_launch(rmsnorm_vec_kernel<TO, V_, T_, false>, dim3(R), dim3(T_), 0, s, x, partial,   \
              parts, part_stride, w, w_bf16, eps, (TO*)y, rows, H)
    if ((R <= 256 && H > 1024) || H > 4 * 256 * 4) {
      const int vec = (H + 4 * 1024 - 1) / (4 * 1024);
      if (vec <= 1) { RMS_GO(1, 1024); }
      else if (vec <= 2) { RMS_GO(2, 1024); }
      else { RMS_GO(4, 1024); }
    } else {
      const int vec = (H + 4 * 256 - 1) / (4 * 256);
      if (vec <= 1) { RMS_GO(1, 256); }
      else if (vec <= 2) { RMS_GO(2, 256); }
      else { RMS_GO(4, 256); }
    }
#undef RMS_GO
    MB_CHECK_LAUNCH("mb_rmsnorm");
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  const size_t smem = parts > 0 ? (size_t)H * sizeof(float) : 0;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel<TW, TO>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MB_FAIL("mb_rmsnorm: a row of %d values: %s", H, cudaGetErrorString(e));
  }
  mb_launch(rmsnorm_kernel<TW, TO>, dim3(R), dim3(threads), smem, s, x, partial, parts, part_stride,
                                                  (const TW*)w, eps, (TO*)y, rows, H);
  MB_CHECK_LAUNCH("mb_rmsnorm");
}

// y[r,:] = w * x[rows ? rows[r] : r, :] / rms. With parts > 0 (rows must be null) the partial
// products are first added into x. y may be null with parts > 0: only the sum into x is done.
MB_EXPORT int mb_rmsnorm(float* x, const float* partial, int parts, long long part_stride,
                         const void* w, int w_dtype, float eps, void* y, int y_dtype,
                         const int* rows, int R, int H, void* stream) {
  if (R <= 0) return 0;
  if (parts > 0 && rows) MB_FAIL("mb_rmsnorm: partial sums with a row gather");
  if (H > 56 * 1024) MB_FAIL("mb_rmsnorm: a row of %d values is not supported (at most 57344)", H);
  cudaStream_t s = (cudaStream_t)stream;
  if (w_dtype == MB_F32 && y_dtype == MB_F32)
    return rmsnorm_launch<float, float>(x, partial, parts, part_stride, w, eps, y, rows, R, H, s);
  if (w_dtype == MB_F32 && y_dtype == MB_BF16)
    return rmsnorm_launch<float, __nv_bfloat16>(x, partial, parts, part_stride, w, eps, y, rows, R, H, s);
  if (w_dtype == MB_BF16 && y_dtype == MB_F32)
    return rmsnorm_launch<__nv_bfloat16, float>(x, partial, parts, part_stride, w, eps, y, rows, R, H, s);
  return rmsnorm_launch<__nv_bfloat16, __nv_bfloat16>(x, partial, parts, part_stride, w, eps, y, rows, R, H, s);
}

// ------------------------------------------------------------------ SwiGLU
// in [T, 2I]: gate in columns [0, I), up in [I, 2I); out [T, I] = f32(g / (1 + exp(-g))) * u
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ in, T* __restrict__ out, size_t total, int I) {
  mb_grid_wait();
  mb_grid_launch_next();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / I;
    const int c = (int)(i - t * I);
    const float g = to_f32<T>(in[t * 2 * I + c]);
    const float u = to_f32<T>(in[t * 2 * I + I + c]);
    const float b = g / (1.0f + expf(-g));
    out[i] = from_f32<T>(b * u);
  }
}

MB_EXPORT int mb_swiglu(const void* in, void* out, int dtype, int T, int I, void* stream) {
  if (T <= 0) return 0;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads
                                                                        : 148 * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == MB_F32)
    mb_launch(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)in, (float*)out, total, I);
  else
    mb_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)in,
                                                             (__nv_bfloat16*)out, total, I);
  MB_CHECK_LAUNCH("mb_swiglu");
}

// ------------------------------------------------------------------ decode without the host
// Between two decode steps that run without a host round trip: the tokens just chosen become
// the next step's input ids and every position moves on by one (and with it what a sequence
// held before the step, which kernels that walk sequences rather than tokens read).
__global__ void advance_decode_kernel(int* __restrict__ tok_ids, int* __restrict__ tok_pos,
                                      const int* __restrict__ chosen, int* __restrict__ history,
                                      int* __restrict__ seq_past, int B) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int t = chosen[b];
  tok_ids[b] = t;
  tok_pos[b] += 1;
  if (seq_past) seq_past[b] += 1;
  if (history) history[b] = t;
}

MB_EXPORT int mb_advance_decode(int* tok_ids, int* tok_pos, const int* chosen, int* history,
                                int* seq_past, int B, void* stream) {
  if (B <= 0) return 0;
  mb_launch(advance_decode_kernel, dim3((B + 127) / 128), dim3(128), 0, (cudaStream_t)stream, tok_ids, tok_pos,
                                                                          chosen, history, seq_past, B);
  MB_CHECK_LAUNCH("mb_advance_decode");
}

// ------------------------------------------------------------------ Dynamic Tanh
// y[r, c] = tanh(alpha * x[src, c]) * w[c] + b[c], value by value in float32: a norm without a
// mean or a variance. alpha is one float32 on the device. As with RMSNorm, `parts` partial
// products [parts][T][H] are first added into the residual row in place, in split order.
// `xb` (or null): a bias [H] that is added into the residual row AFTER y was formed from it:
// the bias of a product that will be accumulated onto that row later (no row gather then).
template <typename TW, typename TO>
__global__ void dynamic_tanh_kernel(float* __restrict__ x, const float* __restrict__ partial,
                                    int parts, size_t part_stride, const TW* __restrict__ w,
                                    const TW* __restrict__ b, const float* __restrict__ alpha,
                                    TO* __restrict__ y, const int* __restrict__ rows, int H,
                                    const TW* __restrict__ xb) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * H;
  const float a = alpha[0];
  TO* yr = y + (size_t)r * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = xr[c];
    if (parts > 0) {
      v += sum_parts(partial + (size_t)src * H + c, parts, part_stride);
      if (!xb) xr[c] = v;
    }
    if (xb) xr[c] = v + to_f32<TW>(xb[c]);
    yr[c] = from_f32<TO>(fmaf(tanhf(a * v), to_f32<TW>(w[c]), to_f32<TW>(b[c])));
  }
}

MB_EXPORT int mb_dynamic_tanh(float* x, const float* partial, int parts, long long part_stride,
                              const void* w, const void* b, int w_dtype, const float* alpha,
                              void* y, int y_dtype, const int* rows, int R, int H, const void* xb,
                              void* stream) {
  if (R <= 0) return 0;
  if ((parts > 0 || xb) && rows) MB_FAIL("mb_dynamic_tanh: sums into the residual with a row gather");
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define GO(TW_, TO_)                                                                          \
  mb_launch(dynamic_tanh_kernel<TW_, TO_>, dim3(R), dim3(threads), 0, s, x, partial, parts,   \
            (size_t)part_stride, (const TW_*)w, (const TW_*)b, alpha, (TO_*)y, rows, H,        \
            (const TW_*)xb)
  if (w_dtype == MB_F32 && y_dtype == MB_F32) GO(float, float);
  else if (w_dtype == MB_F32) GO(float, __nv_bfloat16);
  else if (y_dtype == MB_F32) GO(__nv_bfloat16, float);
  else GO(__nv_bfloat16, __nv_bfloat16);
#undef GO
  MB_CHECK_LAUNCH("mb_dynamic_tanh");
}

// ------------------------------------------------------------------ gated activation
// in [T, 2I]: gate in columns [0, I), up in [I, 2I); out[t, c] = act(g + bg[c]) * (u + bu[c])
// with act = SiLU (0) or the tanh form of GELU (1): 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
// The biases may be null. When `x` is given, the block that handles the first columns of a row
// also adds `xb` [H] into the float32 residual row x[t, :]: the bias of the product that follows
// and accumulates onto that row.
enum { ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_CLAMPED_SWISH = 2 };
__device__ __forceinline__ float act_of(float z, int act) {
  if (act == ACT_GELU_TANH)
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.0f + expf(-z));
}

template <typename T, typename TW>
__global__ void gated_act_kernel(const T* __restrict__ in, T* __restrict__ out, int I, int act,
                                 const TW* __restrict__ bg, const TW* __restrict__ bu,
                                 float* __restrict__ x, const TW* __restrict__ xb, int H,
                                 float limit) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int t = blockIdx.y;
  const T* row = in + (size_t)t * 2 * I;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < I; c += gridDim.x * blockDim.x) {
    float g = to_f32<T>(row[c]), u = to_f32<T>(row[I + c]);
    if (bg) g += to_f32<TW>(bg[c]);
    if (bu) u += to_f32<TW>(bu[c]);
    if (act == ACT_CLAMPED_SWISH) {
      // g' = min(g, limit), u' = clamp(u, -limit, limit): g' sigmoid(1.702 g') (u' + 1)
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      out[(size_t)t * I + c] = from_f32<T>(g / (1.0f + expf(-1.702f * g)) * (u + 1.0f));
    } else {
      out[(size_t)t * I + c] = from_f32<T>(act_of(g, act) * u);
    }
  }
  if (x && blockIdx.x == 0)
    for (int c = threadIdx.x; c < H; c += blockDim.x) x[(size_t)t * H + c] += to_f32<TW>(xb[c]);
}

MB_EXPORT int mb_gated_act(const void* in, void* out, int dtype, int T, int I, int act,
                           const void* bg, const void* bu, int b_dtype, float* x, const void* xb,
                           int H, float limit, void* stream) {
  if (T <= 0) return 0;
  if (act < ACT_SILU || act > ACT_CLAMPED_SWISH) MB_FAIL("mb_gated_act: activation %d", act);
  if ((x == nullptr) != (xb == nullptr)) MB_FAIL("mb_gated_act: x and its bias come together");
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  dim3 grid(max(1, min((I + threads - 1) / threads, 64)), T);
#define GO(T_, TW_)                                                                          \
  mb_launch(gated_act_kernel<T_, TW_>, grid, dim3(threads), 0, s, (const T_*)in, (T_*)out, I, \
            act, (const TW_*)bg, (const TW_*)bu, x, (const TW_*)xb, H, limit)
  if (dtype == MB_F32) {
    if (b_dtype == MB_F32) GO(float, float); else GO(float, __nv_bfloat16);
  } else {
    if (b_dtype == MB_F32) GO(__nv_bfloat16, float); else GO(__nv_bfloat16, __nv_bfloat16);
  }
#undef GO
  MB_CHECK_LAUNCH("mb_gated_act");
}

// ------------------------------------------------------------------ a bias into the residual
template <typename TW>
__global__ void add_bias_kernel(float* __restrict__ x, const TW* __restrict__ b, int H) {
  mb_grid_wait();
  mb_grid_launch_next();
  float* xr = x + (size_t)blockIdx.x * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) xr[c] += to_f32<TW>(b[c]);
}

MB_EXPORT int mb_add_bias(float* x, const void* b, int b_dtype, int T, int H, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (b_dtype == MB_F32) mb_launch(add_bias_kernel<float>, dim3(T), dim3(256), 0, s, x, (const float*)b, H);
  else mb_launch(add_bias_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, s, x, (const __nv_bfloat16*)b, H);
  MB_CHECK_LAUNCH("mb_add_bias");
}

// ------------------------------------------------------------------ what a pass adds
// x[t] += x0[t] + b for a pass through looped layers that starts from the residual plus the
// embedding's output (x0, may be null) plus a vector of the pass (b [H]).
template <typename TW>
__global__ void pass_input_kernel(float* __restrict__ x, const float* __restrict__ x0,
                                  const TW* __restrict__ b, int H) {
  mb_grid_wait();
  mb_grid_launch_next();
  float* xr = x + (size_t)blockIdx.x * H;
  const float* x0r = x0 ? x0 + (size_t)blockIdx.x * H : nullptr;
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    xr[c] = (x0r ? xr[c] + x0r[c] : xr[c]) + to_f32<TW>(b[c]);
}

MB_EXPORT int mb_pass_input(float* x, const float* x0, const void* b, int b_dtype, int T, int H,
                            void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (b_dtype == MB_F32)
    mb_launch(pass_input_kernel<float>, dim3(T), dim3(256), 0, s, x, x0, (const float*)b, H);
  else
    mb_launch(pass_input_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, s, x, x0,
              (const __nv_bfloat16*)b, H);
  MB_CHECK_LAUNCH("mb_pass_input");
}

// ------------------------------------------------------------------ q and k normed as whole rows
// Rows [q (qw) | k (kw) | room (kw)] of ld values: q <- wq * q / rms(q) over all qw values at
// once, k likewise with wk; with copy_k the k values as they came are first copied behind k
// (values that are the keys as projected). Without weights (null) only the copy is made. One block per token; sums in float32.
template <typename T, typename TW>
__global__ void wide_qk_norm_kernel(T* __restrict__ qkv, int ld, int qw, int kw,
                                    const TW* __restrict__ wq, const TW* __restrict__ wk,
                                    float eps, int copy_k) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ float red[33];
  T* row = qkv + (size_t)blockIdx.x * ld;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < qw; c += blockDim.x) {
    const float v = to_f32<T>(row[c]);
    sq = fmaf(v, v, sq);
  }
  for (int c = threadIdx.x; c < kw; c += blockDim.x) {
    const T raw = row[qw + c];
    if (copy_k) row[qw + kw + c] = raw;
    const float v = to_f32<T>(raw);
    sk = fmaf(v, v, sk);
  }
  if (wq == nullptr) return;     // only the copy was asked for
  sq = block_sum(sq, red);
  __syncthreads();
  sk = block_sum(sk, red);
  const float iq = 1.0f / sqrtf(sq / (float)qw + eps), ik = 1.0f / sqrtf(sk / (float)kw + eps);
  for (int c = threadIdx.x; c < qw; c += blockDim.x)
    row[c] = from_f32<T>(to_f32<TW>(wq[c]) * (to_f32<T>(row[c]) * iq));
  for (int c = threadIdx.x; c < kw; c += blockDim.x)
    row[qw + c] = from_f32<T>(to_f32<TW>(wk[c]) * (to_f32<T>(row[qw + c]) * ik));
}

MB_EXPORT int mb_wide_qk_norm(void* qkv, int dtype, int ld, int T, int qw, int kw, const void* wq,
                              const void* wk, int w_dtype, float eps, int copy_k, void* stream) {
  if (T <= 0) return 0;
  if (ld < qw + kw * (copy_k ? 2 : 1)) MB_FAIL("mb_wide_qk_norm: rows of %d values", ld);
  cudaStream_t s = (cudaStream_t)stream;
#define GO(T_, TW_)                                                                            \
  mb_launch(wide_qk_norm_kernel<T_, TW_>, dim3(T), dim3(256), 0, s, (T_*)qkv, ld, qw, kw,       \
            (const TW_*)wq, (const TW_*)wk, eps, copy_k)
  if (dtype == MB_F32) {
    if (w_dtype == MB_F32) GO(float, float); else GO(float, __nv_bfloat16);
  } else {
    if (w_dtype == MB_F32) GO(__nv_bfloat16, float); else GO(__nv_bfloat16, __nv_bfloat16);
  }
#undef GO
  MB_CHECK_LAUNCH("mb_wide_qk_norm");
}

// ------------------------------------------------------------------ a constant factor
__global__ void scale_kernel(float* __restrict__ x, size_t total, float s) {
  mb_grid_wait();
  mb_grid_launch_next();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x)
    x[i] *= s;
}

MB_EXPORT int mb_scale(float* x, long long total, float factor, void* stream) {
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  mb_launch(scale_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, (size_t)total, factor);
  MB_CHECK_LAUNCH("mb_scale");
}

// ------------------------------------------------------------------ a normed sublayer output
// x[t] += w * (y[t] / rms(y[t])) for a sublayer whose output is normed before it joins the
// residual; y is a float32 tensor [T, H] or the sum of `parts` split sums [parts][T][H] of the
// product before (added in split order). `h` (may be null): the new residual row rounded to
// the activation type, which the next sublayer reads. One block per row; sums in float32.
template <typename TW, typename TO>
__global__ void norm_add_kernel(const float* __restrict__ y, int parts, size_t part_stride,
                                const TW* __restrict__ w, float eps, float* __restrict__ x,
                                TO* __restrict__ h, int H) {
  mb_grid_wait();
  mb_grid_launch_next();
  __shared__ float red[33];
  extern __shared__ float rowbuf[];  // H floats
  const int r = blockIdx.x;
  const float* yr = y + (size_t)r * H;
  float sum = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = parts > 1 ? sum_parts(yr + c, parts, part_stride) : yr[c];
    rowbuf[c] = v;
    sum = fmaf(v, v, sum);
  }
  sum = block_sum(sum, red);
  const float inv = 1.0f / sqrtf(sum / (float)H + eps);
  float* xr = x + (size_t)r * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float n = rowbuf[c] * inv;
    const float v = xr[c] + to_f32<TW>(w[c]) * n;
    xr[c] = v;
    if (h) h[(size_t)r * H + c] = from_f32<TO>(v);
  }
}

MB_EXPORT int mb_norm_add(const float* y, int parts, long long part_stride, const void* w,
                          int w_dtype, float eps, float* x, void* h, int h_dtype, int T, int H,
                          void* stream) {
  if (T <= 0) return 0;
  if (parts < 1) MB_FAIL("mb_norm_add: %d parts", parts);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = H >= 2048 ? 512 : H >= 512 ? 256 : 128;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) MB_FAIL("mb_norm_add: rows of %d values", H);
#define GO(TW_, TO_)                                                                         \
  {                                                                                          \
    static size_t configured = 48 * 1024;                                                    \
    if (smem > configured) {                                                                 \
      cudaFuncSetAttribute(norm_add_kernel<TW_, TO_>,                                        \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);         \
      configured = 200 * 1024;                                                               \
    }                                                                                        \
    mb_launch(norm_add_kernel<TW_, TO_>, dim3(T), dim3(threads), smem, s, y, parts,          \
              (size_t)part_stride, (const TW_*)w, eps, x, (TO_*)h, H);                       \
  }
  if (w_dtype == MB_F32) {
    if (h_dtype == MB_F32) GO(float, float) else GO(float, __nv_bfloat16)
  } else {
    if (h_dtype == MB_F32) GO(__nv_bfloat16, float) else GO(__nv_bfloat16, __nv_bfloat16)
  }
#undef GO
  MB_CHECK_LAUNCH("mb_norm_add");
}

// ------------------------------------------------------------------ the residual as an operand
// h = x rounded to the activation type (a sublayer that reads the residual itself).
template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ h, size_t total) {
  mb_grid_wait();
  mb_grid_launch_next();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x)
    h[i] = from_f32<TO>(x[i]);
}

MB_EXPORT int mb_cast_rows(const float* x, void* h, int h_dtype, long long total, void* stream) {
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  if (h_dtype == MB_F32)
    mb_launch(cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x,
              (float*)h, (size_t)total);
  else
    mb_launch(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream,
              x, (__nv_bfloat16*)h, (size_t)total);
  MB_CHECK_LAUNCH("mb_cast_rows");
}

// ------------------------------------------------------------------ an activation of one input
// out[t, c] = act(in[t, c]) (* table[ids[t], col0 + c] when a table is given: a factor that
// the token itself brings), act = SiLU (0), the tanh form of GELU (1) or relu(z)^2 (3).
enum { ACT_RELU_SQUARED = 3 };
template <typename T, typename TW>
__global__ void unary_act_kernel(const T* __restrict__ in, int ld_in, T* __restrict__ out, int N,
                                 int act, const TW* __restrict__ table, int ld_table, int col0,
                                 const int* __restrict__ ids, int V) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int t = blockIdx.y;
  const T* row = in + (size_t)t * ld_in;
  const TW* trow = nullptr;
  if (table) {
    int id = ids[t];
    if (id < 0 || id >= V) id = 0;  // the host refuses such ids before the step
    trow = table + (size_t)id * ld_table + col0;
  }
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < N; c += gridDim.x * blockDim.x) {
    const float z = to_f32<T>(row[c]);
    float a;
    if (act == ACT_RELU_SQUARED) {
      const float p = fmaxf(z, 0.f);
      a = p * p;
    } else {
      a = act_of(z, act);
    }
    if (trow) a *= to_f32<TW>(trow[c]);
    out[(size_t)t * N + c] = from_f32<T>(a);
  }
}

MB_EXPORT int mb_unary_act(const void* in, int ld_in, void* out, int dtype, int T, int N, int act,
                           const void* table, int table_dtype, int ld_table, int col0,
                           const int* ids, int V, void* stream) {
  if (T <= 0 || N <= 0) return 0;
  if (act != ACT_SILU && act != ACT_GELU_TANH && act != ACT_RELU_SQUARED)
    MB_FAIL("mb_unary_act: activation %d", act);
  if (table != nullptr && ids == nullptr) MB_FAIL("mb_unary_act: a table without token ids");
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = N >= 256 ? 256 : 64;
  dim3 grid(max(1, min((N + threads - 1) / threads, 64)), T);
#define GO(T_, TW_)                                                                           \
  mb_launch(unary_act_kernel<T_, TW_>, grid, dim3(threads), 0, s, (const T_*)in, ld_in,        \
            (T_*)out, N, act, (const TW_*)table, ld_table, col0, ids, V)
  if (dtype == MB_F32) {
    if (table_dtype == MB_F32) GO(float, float); else GO(float, __nv_bfloat16);
  } else {
    if (table_dtype == MB_F32) GO(__nv_bfloat16, float); else GO(__nv_bfloat16, __nv_bfloat16);
  }
#undef GO
  MB_CHECK_LAUNCH("mb_unary_act");
}

// ------------------------------------------------------------------ a soft cap
// x = cap * tanh(x / cap), float32 in place (logits).
__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap) {
  mb_grid_wait();
  mb_grid_launch_next();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

MB_EXPORT int mb_softcap(float* x, long long total, float cap, void* stream) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) MB_FAIL("mb_softcap: a cap of %g", (double)cap);
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  mb_launch(softcap_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, (size_t)total,
            cap);
  MB_CHECK_LAUNCH("mb_softcap");
}
