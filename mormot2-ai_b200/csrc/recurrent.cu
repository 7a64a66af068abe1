// Recurrent mixers: what runs token after token over a state of fixed size per sequence.
// The state lives in float32 in the engine's state arena ([slots][state_stride] floats; a
// mixer's part of a slot's row starts at `state_off`), is read when a step begins and written
// when it ends, so a sequence may be fed in portions of any size. Everything that enters a
// recurrence is float32: decays, gates, maxima, norms. One block per (sequence, head) walks the
// step's tokens of its sequence in order, sixteen at a time staged in shared memory; a thread
// owns one value column of the head's matrix state, which is kept in shared memory.
//
//   token_shift   [h[t] ; h[t-1] - h[t]], from which every blend h + (h' - h) mu_s is projected
//                 by one product; h[-1] of a sequence is kept in the state (zeros at first)
//   wkv_scan      decay w = exp(-exp(lw + w0)); o_t = (S + diag(u) k v^T)^T r;
//                 S <- diag(w) S + k v^T; then o / rms(o) * norm * silu(g) per head
//   mlstm_scan    log gates i = cap tanh((zi + bi)/cap), f = logsigmoid(cap tanh((zf + bf)/cap));
//                 m' = max(f + m, i); S <- e^(f+m-m') S + e^(i-m') k v^T; n likewise with k;
//                 o = S^T q / (max(|n.q|, e^(-m')) + 1e-6); then o / rms(o) * norm * sigmoid(g)
//   retention_scan  q, k turned by the position; S <- decay S + (k / sqrt(D)) v^T; o = S^T q;
//                 then o / rms(o) * silu(g)
//   retention_chunked  the same recurrence chunk by chunk (three kernels) for a step that
//                 brings many tokens of a sequence
#include "common.cuh"

MB_DEFINE_LAST_ERROR

// ------------------------------------------------------------------ token shift
// out[t] = [h[t] ; h[t-1] - h[t]] (2 W values): a projection of a blend h + (h' - h) mu is then
// ONE product of this row with the weight [W_s | W_s diag(mu_s)], for all blends s at once.
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ h, const float* __restrict__ state,
                                   size_t state_stride, size_t state_off,
                                   const int* __restrict__ tok_seq,
                                   const int* __restrict__ seq_start,
                                   const int* __restrict__ seq_slot, T* __restrict__ out, int W) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  const bool first = seq_start[b] == t;
  const float* prev_state = state + (size_t)seq_slot[b] * state_stride + state_off;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const T hv = h[(size_t)t * W + c];
    const float pv = first ? prev_state[c] : to_f32<T>(h[(size_t)(t - 1) * W + c]);
    out[(size_t)t * 2 * W + c] = hv;
    out[(size_t)t * 2 * W + W + c] = from_f32<T>(pv - to_f32<T>(hv));
  }
}

MB_EXPORT int mb_token_shift(const void* h, int dtype, const float* state, long long state_stride,
                             long long state_off, const int* tok_seq, const int* seq_start,
                             const int* seq_slot, void* out, int T, int W, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = W >= 1024 ? 256 : 128;
  if (dtype == MB_F32)
    mb_launch(token_shift_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)h, state,
              (size_t)state_stride, (size_t)state_off, tok_seq, seq_start, seq_slot,
              (float*)out, W);
  else
    mb_launch(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s,
              (const __nv_bfloat16*)h, state, (size_t)state_stride, (size_t)state_off, tok_seq,
              seq_start, seq_slot, (__nv_bfloat16*)out, W);
  MB_CHECK_LAUNCH("mb_token_shift");
}

// ------------------------------------------------------------------ the walks over the tokens
// A block owns a slice of a head's value columns (all of them where the batch gives blocks
// enough; else the columns are dealt over several blocks so that a single prompt does not
// leave most multiprocessors idle, and the heads' unit norm runs as a kernel after). It
// stages SCAN_CT tokens of its head's inputs in shared memory at once (all loads in flight
// together) and walks them without a barrier between tokens: P groups of threads share the
// rows of a column, a thread keeps its rows of its column in registers (R of them at most;
// R = 0: more than 32, the state then lies in shared memory) and reads the staged vectors.
#define SCAN_CT 16

__device__ __forceinline__ int pad32(int v) { return (v + 31) & ~31; }

// r, k, v, lw, g: float32 [T, ld] each (head hd's values at column hd * D + i); w0, u, normw:
// float32 [H * D]. State of a slot: [W values of the last h | H x D x D]. out [T, H * D] (one
// slice of columns a head: normed and gated here); raw [T, H * D] float32 (several slices: the
// outputs as they are, for head_norm_gate_kernel).
template <typename T, int R>
__global__ void __launch_bounds__(512, 1)
wkv_scan_kernel(const float* __restrict__ r, const float* __restrict__ k,
                const float* __restrict__ v, const float* __restrict__ lw,
                const float* __restrict__ g, int ld, const float* __restrict__ w0,
                const float* __restrict__ u, const float* __restrict__ normw, float eps,
                float* __restrict__ state, size_t state_stride, size_t state_off,
                const T* __restrict__ h, int W, const int* __restrict__ seq_start,
                const int* __restrict__ seq_slot, T* __restrict__ out, float* __restrict__ raw,
                int H, int D) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) float wk_smem[];
  const int NS = gridDim.z, CW = (D + NS - 1) / NS;
  const int c0 = blockIdx.z * CW, cw = max(0, min(D, c0 + CW) - c0);
  const int Cp = pad32(CW), P = blockDim.x / Cp;
  const int part = threadIdx.x / Cp, j = threadIdx.x - part * Cp;
  const int per = (D + P - 1) / P, i0 = min(D, part * per), cnt = min(D, i0 + per) - i0;
  float* S = wk_smem;                                  // [D][CW] (R = 0 only)
  float4* vec = (float4*)(S + (R > 0 ? 0 : ((D * CW + 3) & ~3)));   // [CT][D]: r, k, decay, u k
  float* sv = (float*)(vec + SCAN_CT * D + 64);        // [CT][CW] v (64 entries of room behind
                                                       // vec: a thread may read past its rows)
  float* sg = sv + SCAN_CT * CW;                       // [CT][CW] g
  float* so = sg + SCAN_CT * CW;                       // [CT][P][CW] o, summed over a part's rows
  const int b = blockIdx.x, hd = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  float* st = state + (size_t)seq_slot[b] * state_stride + state_off;
  float* Sg = st + W + (size_t)hd * D * D + c0;        // row i of this slice at Sg + i * D
  const bool own = j < cw && part < P;
  float Sr[R > 0 ? R : 1];
  if (R > 0) {
#pragma unroll
    for (int q = 0; q < (R > 0 ? R : 1); ++q)
      Sr[q] = (own && q < cnt) ? Sg[(size_t)(i0 + q) * D + j] : 0.f;
  } else {
    for (int e = threadIdx.x; e < D * cw; e += blockDim.x) {
      const int i = e / cw, jj = e - i * cw;
      S[i * CW + jj] = Sg[(size_t)i * D + jj];
    }
  }
  for (int c = 0; c < n; c += SCAN_CT) {
    const int cn = min(SCAN_CT, n - c);
    for (int e = threadIdx.x; e < cn * D; e += blockDim.x) {
      const int tt = e / D, i = e - tt * D;
      const size_t at = (size_t)(t0 + c + tt) * ld + hd * D + i;
      const float kk = k[at];
      vec[e] = make_float4(r[at], kk, expf(-expf(lw[at] + w0[hd * D + i])), u[hd * D + i] * kk);
    }
    for (int e = threadIdx.x; e < cn * cw; e += blockDim.x) {
      const int tt = e / cw, jj = e - tt * cw;
      const size_t at = (size_t)(t0 + c + tt) * ld + hd * D + c0 + jj;
      sv[tt * CW + jj] = v[at];
      sg[tt * CW + jj] = g[at];
    }
    __syncthreads();
    if (own) {
      for (int tt = 0; tt < cn; ++tt) {
        const float vj = sv[tt * CW + j];
        const float4* x = vec + tt * D;
        float o = 0.f;
        if (R > 0) {
          float o4[4] = {0.f, 0.f, 0.f, 0.f};     // four sums side by side: shorter chains
#pragma unroll
          for (int q = 0; q < (R > 0 ? R : 1); ++q) {
            // no branch: rows past this thread's last are read (they exist) and left out
            const float4 xi = x[i0 + q];
            const float sc = Sr[q];
            const float with = fmaf(xi.x, fmaf(xi.w, vj, sc), o4[q & 3]);
            o4[q & 3] = q < cnt ? with : o4[q & 3];
            Sr[q] = fmaf(xi.z, sc, xi.y * vj);
          }
          o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
        } else {
          // eight rows at a time: their loads are asked for together, then the multiply-adds,
          // then the stores (written one by one a store would hold the next load back)
          for (int ib = i0; ib < i0 + cnt; ib += 8) {
            float4 xi[8];
            float sc[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int i = min(ib + q, i0 + cnt - 1);
              xi[q] = x[i];
              sc[q] = S[i * CW + j];
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              if (ib + q < i0 + cnt) {
                o = fmaf(xi[q].x, fmaf(xi[q].w, vj, sc[q]), o);
                S[(ib + q) * CW + j] = fmaf(xi[q].z, sc[q], xi[q].y * vj);
              }
            }
          }
        }
        so[(tt * P + part) * CW + j] = o;
      }
    }
    __syncthreads();
    if (raw != nullptr) {
      for (int e = threadIdx.x; e < cn * cw; e += blockDim.x) {
        const int tt = e / cw, jj = e - tt * cw;
        float o = 0.f;
        for (int pp = 0; pp < P; ++pp) o += so[(tt * P + pp) * CW + jj];
        raw[(size_t)(t0 + c + tt) * H * D + hd * D + c0 + jj] = o;
      }
    } else {
      // one slice: the head's unit norm, its weight and the gate here, a warp a token
      for (int tt = warp; tt < cn; tt += warps) {
        float ov[8];   // heads of up to 256 values a lane's eight; beyond, the sums are formed again
        float ss = 0.f;
        for (int i = lane, q = 0; i < D; i += 32, ++q) {
          float o = 0.f;
          for (int pp = 0; pp < P; ++pp) o += so[(tt * P + pp) * CW + i];
          if (q < 8) ov[q] = o;
          ss = fmaf(o, o, ss);
        }
        const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
        T* orow = out + (size_t)(t0 + c + tt) * H * D + hd * D;
        for (int i = lane, q = 0; i < D; i += 32, ++q) {
          float o = 0.f;
          if (q < 8) {
            o = ov[q];
          } else {
            for (int pp = 0; pp < P; ++pp) o += so[(tt * P + pp) * CW + i];
          }
          const float gi = sg[tt * CW + i];
          orow[i] = from_f32<T>(o * inv * normw[hd * D + i] * (gi / (1.0f + expf(-gi))));
        }
      }
    }
    __syncthreads();
  }
  if (R > 0) {
#pragma unroll
    for (int q = 0; q < (R > 0 ? R : 1); ++q)
      if (own && q < cnt) Sg[(size_t)(i0 + q) * D + j] = Sr[q];
  } else {
    for (int e = threadIdx.x; e < D * cw; e += blockDim.x) {
      const int i = e / cw, jj = e - i * cw;
      Sg[(size_t)i * D + jj] = S[i * CW + jj];
    }
  }
  if (hd == 0 && blockIdx.z == 0 && n > 0)
    for (int cc = threadIdx.x; cc < W; cc += blockDim.x)
      st[cc] = to_f32<T>(h[(size_t)(t0 + n - 1) * W + cc]);
}

// out[t, hd, :] = o / rms(o) * normw * gate(g) for every token and head, a warp each (normw
// null: ones); o: raw
// [T, H * DV] float32; g: the gates' logits, head hd of token t at g + t * ldg + hd * DV;
// gate 0: g sigmoid(g), 1: sigmoid(g).
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ raw, const float* __restrict__ g,
                                      int ldg, const float* __restrict__ normw, float eps,
                                      int gate, T* __restrict__ out, int rows, int H, int DV) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= rows) return;
  const int t = idx / H, hd = idx - t * H;
  const float* o = raw + (size_t)idx * DV;
  const float* gg = g + (size_t)t * ldg + hd * DV;
  float ss = 0.f;
  for (int i = lane; i < DV; i += 32) ss = fmaf(o[i], o[i], ss);
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)DV + eps);
  for (int i = lane; i < DV; i += 32) {
    const float gi = gg[i], sig = 1.0f / (1.0f + expf(-gi));
    const float w = normw ? normw[hd * DV + i] : 1.0f;
    out[(size_t)idx * DV + i] = from_f32<T>(o[i] * inv * w * (gate ? sig : gi * sig));
  }
}

template <typename T>
static void launch_head_norm(const float* raw, const float* g, int ldg, const float* normw,
                             float eps, int gate, void* out, int T_, int H, int DV,
                             cudaStream_t s) {
  const int rows = T_ * H;
  mb_launch(head_norm_gate_kernel<T>, dim3((rows + 3) / 4), dim3(128), 0, s, raw, g, ldg, normw,
            eps, gate, (T*)out, rows, H, DV);
}

// how many groups of threads share a column's rows: as many as keep a block within 512
// threads, at most 8
static int scan_parts(int columns) {
  const int cp = (columns + 31) / 32 * 32;
  int p = 512 / cp;
  return p < 1 ? 1 : (p > 8 ? 8 : p);
}

// the rows of a state column that one thread has: 8, 16 or 32 in registers, 0: more, the
// state stays in shared memory
static int scan_rows(int D, int columns) {
  const int P = scan_parts(columns), per = (D + P - 1) / P;
  return per <= 8 ? 8 : per <= 16 ? 16 : per <= 32 ? 32 : 0;
}

// Over how many blocks a head's DV value columns (of D rows) are dealt: one while the step has
// 96 (sequence, head) pairs or more (a decode step of a batch), else doubled while a slice
// holds more than 4,096 values of the state (measured: below that a block's time is the
// chunks' fixed cost, and more blocks gain nothing), keeps 32 columns and the block
// `need_threads` threads. It depends on the step's shape only.
static int scan_slices(int B, int H, int D, int DV, int need_threads) {
  int ns = 1;
  while (B * H * ns < 96 && D * ((DV + ns - 1) / ns) > 4096) {
    const int cw = (DV + 2 * ns - 1) / (2 * ns);
    if (cw < 32 || ((cw + 31) / 32 * 32) * scan_parts(cw) < need_threads) break;
    ns *= 2;
  }
  return ns;
}

static size_t wkv_smem_bytes(int D, int CW) {
  const size_t state = scan_rows(D, CW) ? 0 : (size_t)((D * CW + 3) & ~3);
  return (state + (size_t)SCAN_CT * (4 * D + CW * (2 + scan_parts(CW))) + 64 * 4) * sizeof(float);
}

// `raw`: float32 [T, H * D] of scratch, used when a head's columns are dealt over several blocks.
MB_EXPORT int mb_wkv_scan(const float* r, const float* k, const float* v, const float* lw,
                          const float* g, int ld, const float* w0, const float* u,
                          const float* normw, float eps, float* state, long long state_stride,
                          long long state_off, const void* h, int dtype, int W,
                          const int* seq_start, const int* seq_slot, void* out, float* raw,
                          int T_, int B, int H, int D, void* stream) {
  if (B <= 0) return 0;
  if (D <= 0 || D > 512) MB_FAIL("mb_wkv_scan: heads of %d values (at most 512)", D);
  const int NS = raw ? scan_slices(B, H, D, D, 32) : 1;
  const int CW = (D + NS - 1) / NS;
  const size_t smem = wkv_smem_bytes(D, CW);
  if (smem > 200 * 1024)
    MB_FAIL("mb_wkv_scan: heads of %d values (what a block stages must fit 200 KB)", D);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = (CW + 31) / 32 * 32 * scan_parts(CW);
  float* raw_used = NS > 1 ? raw : nullptr;
#define GO(T_t, R_)                                                                            \
  {                                                                                            \
    static size_t configured = 48 * 1024;                                                      \
    if (smem > configured) {                                                                   \
      cudaFuncSetAttribute(wkv_scan_kernel<T_t, R_>,                                           \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
      configured = 200 * 1024;                                                                 \
    }                                                                                          \
    mb_launch(wkv_scan_kernel<T_t, R_>, dim3(B, H, NS), dim3(threads), smem, s, r, k, v, lw, g, \
              ld, w0, u, normw, eps, state, (size_t)state_stride, (size_t)state_off,           \
              (const T_t*)h, W, seq_start, seq_slot, (T_t*)out, raw_used, H, D);               \
    if (NS > 1) launch_head_norm<T_t>(raw, g, ld, normw, eps, 0, out, T_, H, D, s);            \
  }
#define GOR(T_t)                                                                               \
  switch (scan_rows(D, CW)) {                                                                  \
    case 8: GO(T_t, 8) break;                                                                  \
    case 16: GO(T_t, 16) break;                                                                \
    case 32: GO(T_t, 32) break;                                                                \
    default: GO(T_t, 0)                                                                        \
  }
  if (dtype == MB_F32) GOR(float) else GOR(__nv_bfloat16)
#undef GOR
#undef GO
  MB_CHECK_LAUNCH("mb_wkv_scan");
}

// ------------------------------------------------------------------ matrix memory with gates
// z: float32 [T, ld], the fused projection: q at column cq + hd * D, k at ck + hd * D, v at
// cv + hd * DV, the output gate at cg + hd * DV, the input and forget gates at ci + hd and
// cf + hd. bi, bf: float32 [H]. normw: float32 [H * DV]. State of a slot, per head:
// [D x DV | D of n | m]. out / raw as in wkv_scan_kernel (raw holds S^T q over its denominator).
__device__ __forceinline__ float log_sigmoid(float x) {
  return fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
}

template <typename T, int R>
__global__ void __launch_bounds__(512, 1)
mlstm_scan_kernel(const float* __restrict__ z, int ld, int cq, int ck, int cv, int cg, int ci,
                  int cf, const float* __restrict__ bi, const float* __restrict__ bf, float cap,
                  float q_scale, const float* __restrict__ normw, float eps,
                  float* __restrict__ state, size_t state_stride, size_t state_off,
                  const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                  T* __restrict__ out, float* __restrict__ raw, int H, int D, int DV) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) float ml_smem[];
  const int NS = gridDim.z, CW = (DV + NS - 1) / NS;
  const int c0 = blockIdx.z * CW, cw = max(0, min(DV, c0 + CW) - c0);
  // one slice: the block is as wide as the larger of D and DV (a thread a normalizer value)
  const int Cp = NS == 1 ? pad32(max(D, DV)) : pad32(CW), P = blockDim.x / Cp;
  const int part = threadIdx.x / Cp, j = threadIdx.x - part * Cp;
  const int per = (D + P - 1) / P, i0 = min(D, part * per), cnt = min(D, i0 + per) - i0;
  float* S = ml_smem;                                   // [D][CW] (R = 0 only)
  float2* qk = (float2*)(S + (R > 0 ? 0 : ((D * CW + 3) & ~3)));   // [CT][D]: q (scaled), k
  float* sv = (float*)(qk + SCAN_CT * D + 64);          // [CT][CW] v (64 entries of room behind qk)
  float* sg = sv + SCAN_CT * CW;                        // [CT][CW] the output gate's logit
  float* snq = sg + SCAN_CT * CW;                       // [CT][D] n_i q_i
  float* sab = snq + SCAN_CT * D;                       // [CT][4]: the state's factor, the
                                                        // input's, e^(-m), the denominator
  float* snum = sab + SCAN_CT * 4;                      // [CT][P][CW] S^T q, summed over a part's rows
  const int b = blockIdx.x, hd = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  float* st = state + (size_t)seq_slot[b] * state_stride + state_off +
              (size_t)hd * ((size_t)D * DV + D + 1);
  float* Sg = st + c0;                                  // row i of this slice at Sg + i * DV
  const bool own_v = j < cw && part < P, own_k = (int)threadIdx.x < D;
  float Sr[R > 0 ? R : 1];
  if (R > 0) {
#pragma unroll
    for (int q = 0; q < (R > 0 ? R : 1); ++q)
      Sr[q] = (own_v && q < cnt) ? Sg[(size_t)(i0 + q) * DV + j] : 0.f;
  } else {
    for (int e = threadIdx.x; e < D * cw; e += blockDim.x) {
      const int i = e / cw, jj = e - i * cw;
      S[i * CW + jj] = Sg[(size_t)i * DV + jj];
    }
  }
  // every slice keeps the whole normalizer and the running maximum (they need all of k); the
  // first one writes them back
  float nj = own_k ? st[(size_t)D * DV + threadIdx.x] : 0.f;
  float m = st[(size_t)D * DV + D];          // the last thread's copy is the one that counts
  const float bih = bi[hd], bfh = bf[hd];
  for (int c = 0; c < n; c += SCAN_CT) {
    const int cn = min(SCAN_CT, n - c);
    for (int e = threadIdx.x; e < cn * D; e += blockDim.x) {
      const int tt = e / D, i = e - tt * D;
      const float* zr = z + (size_t)(t0 + c + tt) * ld;
      qk[e] = make_float2(zr[cq + hd * D + i] * q_scale, zr[ck + hd * D + i]);
    }
    for (int e = threadIdx.x; e < cn * cw; e += blockDim.x) {
      const int tt = e / cw, jj = e - tt * cw;
      const float* zr = z + (size_t)(t0 + c + tt) * ld;
      sv[tt * CW + jj] = zr[cv + hd * DV + c0 + jj];
      sg[tt * CW + jj] = zr[cg + hd * DV + c0 + jj];
    }
    if (warp == warps - 1) {
      // the gates by the last warp: every token's two logarithms side by side (a lane a
      // token), then the running maximum token after token by one lane (additions and maxima
      // only), then the exponentials side by side again
      float gi = 0.f, gf = 0.f;
      if (lane < cn) {
        const float* zr = z + (size_t)(t0 + c + lane) * ld;
        gi = cap * tanhf((zr[ci + hd] + bih) / cap);
        gf = log_sigmoid(cap * tanhf((zr[cf + hd] + bfh) / cap));
        sab[lane * 4] = gi;
        sab[lane * 4 + 1] = gf;
      }
      __syncwarp();
      if (lane == 31) {
        for (int tt = 0; tt < cn; ++tt) {
          const float m_new = fmaxf(sab[tt * 4 + 1] + m, sab[tt * 4]);
          sab[tt * 4 + 2] = m;          // the maximum before this token
          sab[tt * 4 + 3] = m_new;
          m = m_new;
        }
      }
      __syncwarp();
      if (lane < cn) {
        const float m_old = sab[lane * 4 + 2], m_new = sab[lane * 4 + 3];
        sab[lane * 4] = expf(gf + m_old - m_new);
        sab[lane * 4 + 1] = expf(gi - m_new);
        sab[lane * 4 + 2] = expf(-m_new);
      }
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float a = sab[tt * 4], bb = sab[tt * 4 + 1];
      if (own_k) {
        const float2 x = qk[tt * D + threadIdx.x];
        nj = fmaf(a, nj, bb * x.y);
        snq[tt * D + threadIdx.x] = nj * x.x;
      }
      if (own_v) {
        const float bv = bb * sv[tt * CW + j];
        const float2* x = qk + tt * D;
        float num = 0.f;
        if (R > 0) {
          float n4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int q = 0; q < (R > 0 ? R : 1); ++q) {
            const float2 xi = x[i0 + q];      // no branch, as in wkv_scan_kernel
            const float s = fmaf(a, Sr[q], xi.y * bv);
            Sr[q] = s;
            const float with = fmaf(s, xi.x, n4[q & 3]);
            n4[q & 3] = q < cnt ? with : n4[q & 3];
          }
          num = (n4[0] + n4[1]) + (n4[2] + n4[3]);
        } else {
          for (int ib = i0; ib < i0 + cnt; ib += 8) {   // eight rows at a time, as in wkv_scan_kernel
            float2 xi[8];
            float sc[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int i = min(ib + q, i0 + cnt - 1);
              xi[q] = x[i];
              sc[q] = S[i * CW + j];
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              if (ib + q < i0 + cnt) {
                const float s = fmaf(a, sc[q], xi[q].y * bv);
                S[(ib + q) * CW + j] = s;
                num = fmaf(s, xi[q].x, num);
              }
            }
          }
        }
        snum[(tt * P + part) * CW + j] = num;
      }
    }
    __syncthreads();
    if (raw != nullptr) {
      for (int tt = warp; tt < cn; tt += warps) {
        float nq = 0.f;
        for (int i = lane; i < D; i += 32) nq += snq[tt * D + i];
        nq = warp_sum(nq);
        if (lane == 0) sab[tt * 4 + 3] = fmaxf(fabsf(nq), sab[tt * 4 + 2]) + 1e-6f;
      }
      __syncthreads();
      for (int e = threadIdx.x; e < cn * cw; e += blockDim.x) {
        const int tt = e / cw, jj = e - tt * cw;
        float num = 0.f;
        for (int pp = 0; pp < P; ++pp) num += snum[(tt * P + pp) * CW + jj];
        raw[(size_t)(t0 + c + tt) * H * DV + hd * DV + c0 + jj] = num / sab[tt * 4 + 3];
      }
    } else {
      for (int tt = warp; tt < cn; tt += warps) {
        float nv[8];   // value rows of up to 256 a lane's eight; beyond, the sums are formed again
        float nq = 0.f, ss = 0.f;
        for (int i = lane; i < D; i += 32) nq += snq[tt * D + i];
        for (int i = lane, q = 0; i < DV; i += 32, ++q) {
          float num = 0.f;
          for (int pp = 0; pp < P; ++pp) num += snum[(tt * P + pp) * CW + i];
          if (q < 8) nv[q] = num;
          ss = fmaf(num, num, ss);
        }
        nq = warp_sum(nq);
        ss = warp_sum(ss);
        const float den = fmaxf(fabsf(nq), sab[tt * 4 + 2]) + 1e-6f;
        const float inv = 1.0f / sqrtf(ss / (den * den) / (float)DV + eps);
        T* orow = out + (size_t)(t0 + c + tt) * H * DV + hd * DV;
        for (int i = lane, q = 0; i < DV; i += 32, ++q) {
          float num = 0.f;
          if (q < 8) {
            num = nv[q];
          } else {
            for (int pp = 0; pp < P; ++pp) num += snum[(tt * P + pp) * CW + i];
          }
          const float gate = 1.0f / (1.0f + expf(-sg[tt * CW + i]));
          orow[i] = from_f32<T>(num / den * inv * normw[hd * DV + i] * gate);
        }
      }
    }
    __syncthreads();
  }
  if (R > 0) {
#pragma unroll
    for (int q = 0; q < (R > 0 ? R : 1); ++q)
      if (own_v && q < cnt) Sg[(size_t)(i0 + q) * DV + j] = Sr[q];
  } else {
    for (int e = threadIdx.x; e < D * cw; e += blockDim.x) {
      const int i = e / cw, jj = e - i * cw;
      Sg[(size_t)i * DV + jj] = S[i * CW + jj];
    }
  }
  if (blockIdx.z == 0) {
    if (own_k) st[(size_t)D * DV + threadIdx.x] = nj;
    if (threadIdx.x == blockDim.x - 1) st[(size_t)D * DV + D] = m;
  }
}

static size_t mlstm_smem_bytes(int D, int CW, int P, int R) {
  const size_t state = R ? 0 : (size_t)((D * CW + 3) & ~3);
  return (state + (size_t)SCAN_CT * (3 * D + (2 + P) * CW + 4) + 64 * 2) * sizeof(float);
}

MB_EXPORT int mb_mlstm_scan(const float* z, int ld, int cq, int ck, int cv, int cg, int ci, int cf,
                            const float* bi, const float* bf, float cap, float q_scale,
                            const float* normw, float eps, float* state, long long state_stride,
                            long long state_off, const int* seq_start, const int* seq_slot,
                            void* out, float* raw, int dtype, int T_, int B, int H, int D, int DV,
                            void* stream) {
  if (B <= 0) return 0;
  if (D <= 0 || DV <= 0 || D > 512 || DV > 512)
    MB_FAIL("mb_mlstm_scan: heads of %d x %d values (at most 512 each)", D, DV);
  const int NS = raw ? scan_slices(B, H, D, DV, D) : 1;
  const int CW = (DV + NS - 1) / NS;
  // one slice: a block as wide as the larger of D and DV; several: as wide as the slice
  const int width = NS == 1 ? (D > DV ? D : DV) : CW;
  const int P = scan_parts(width), per = (D + P - 1) / P;
  const int R = per <= 8 ? 8 : per <= 16 ? 16 : per <= 32 ? 32 : 0;
  const size_t smem = mlstm_smem_bytes(D, CW, P, R);
  if (smem > 200 * 1024)
    MB_FAIL("mb_mlstm_scan: heads of %d x %d values (what a block stages must fit 200 KB)", D, DV);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = (width + 31) / 32 * 32 * P;
  float* raw_used = NS > 1 ? raw : nullptr;
#define GO(T_t, R_)                                                                            \
  {                                                                                            \
    static size_t configured = 48 * 1024;                                                      \
    if (smem > configured) {                                                                   \
      cudaFuncSetAttribute(mlstm_scan_kernel<T_t, R_>,                                         \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
      configured = 200 * 1024;                                                                 \
    }                                                                                          \
    mb_launch(mlstm_scan_kernel<T_t, R_>, dim3(B, H, NS), dim3(threads), smem, s, z, ld, cq,   \
              ck, cv, cg, ci, cf, bi, bf, cap, q_scale, normw, eps, state,                     \
              (size_t)state_stride, (size_t)state_off, seq_start, seq_slot, (T_t*)out,         \
              raw_used, H, D, DV);                                                             \
    if (NS > 1) launch_head_norm<T_t>(raw, z + cg, ld, normw, eps, 1, out, T_, H, DV, s);      \
  }
#define GOR(T_t)                                                                               \
  switch (R) {                                                                                 \
    case 8: GO(T_t, 8) break;                                                                  \
    case 16: GO(T_t, 16) break;                                                                \
    case 32: GO(T_t, 32) break;                                                                \
    default: GO(T_t, 0)                                                                        \
  }
  if (dtype == MB_F32) GOR(float) else GOR(__nv_bfloat16)
#undef GOR
#undef GO
  MB_CHECK_LAUNCH("mb_mlstm_scan");
}

// ------------------------------------------------------------------ retention
// Linear attention with a constant decay per head and no denominator. z: float32 [T, ld], the
// fused projection: q at column cq + hd * D, k at ck + hd * D, v at cv + hd * DV, the output
// gate's logit at cg + hd * DV. q and k turn by the token's position in the rotate-half pairing
// over their first rot_dim values (angle = f32(inv_freq[i] * pos)); k is then multiplied by
// k_scale. S <- decay[hd] S + k v^T; o = S^T q (the state after the token); then
// o / rms(o) * silu(g). State of a slot, per head: D x DV. out / raw as in wkv_scan_kernel.
template <typename T, int R>
__global__ void __launch_bounds__(512, 1)
retention_scan_kernel(const float* __restrict__ z, int ld, int cq, int ck, int cv, int cg,
                      const float* __restrict__ decay, float k_scale,
                      const float* __restrict__ inv_freq, int rot_dim,
                      const int* __restrict__ tok_pos, float eps, float* __restrict__ state,
                      size_t state_stride, size_t state_off, const int* __restrict__ seq_start,
                      const int* __restrict__ seq_slot, T* __restrict__ out,
                      float* __restrict__ raw, int H, int D, int DV) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) float rt_smem[];
  const int NS = gridDim.z, CW = (DV + NS - 1) / NS;
  const int c0 = blockIdx.z * CW, cw = max(0, min(DV, c0 + CW) - c0);
  const int Cp = pad32(CW), P = blockDim.x / Cp;
  const int part = threadIdx.x / Cp, j = threadIdx.x - part * Cp;
  const int per = (D + P - 1) / P, i0 = min(D, part * per), cnt = min(D, i0 + per) - i0;
  float* S = rt_smem;                                   // [D][CW] (R = 0 only)
  float2* qk = (float2*)(S + (R > 0 ? 0 : ((D * CW + 3) & ~3)));   // [CT][D]: q, k (turned, scaled)
  float* sv = (float*)(qk + SCAN_CT * D + 64);          // [CT][CW] v (64 entries of room behind qk)
  float* sg = sv + SCAN_CT * CW;                        // [CT][CW] the output gate's logit
  float* snum = sg + SCAN_CT * CW;                      // [CT][P][CW] S^T q, summed over a part's rows
  const int b = blockIdx.x, hd = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  float* Sg = state + (size_t)seq_slot[b] * state_stride + state_off +
              (size_t)hd * D * DV + c0;                 // row i of this slice at Sg + i * DV
  const bool own = j < cw && part < P;
  const float a = decay[hd];
  const int half = rot_dim >> 1;
  float Sr[R > 0 ? R : 1];
  if (R > 0) {
#pragma unroll
    for (int q = 0; q < (R > 0 ? R : 1); ++q)
      Sr[q] = (own && q < cnt) ? Sg[(size_t)(i0 + q) * DV + j] : 0.f;
  } else {
    for (int e = threadIdx.x; e < D * cw; e += blockDim.x) {
      const int i = e / cw, jj = e - i * cw;
      S[i * CW + jj] = Sg[(size_t)i * DV + jj];
    }
  }
  for (int c = 0; c < n; c += SCAN_CT) {
    const int cn = min(SCAN_CT, n - c);
    for (int e = threadIdx.x; e < cn * D; e += blockDim.x) {
      const int tt = e / D, i = e - tt * D;
      const float* zr = z + (size_t)(t0 + c + tt) * ld;
      float qv = zr[cq + hd * D + i], kv = zr[ck + hd * D + i];
      if (i < rot_dim) {
        const bool lo = i < half;
        const int f = lo ? i : i - half, other = lo ? i + half : i - half;
        const float angle = inv_freq[f] * (float)tok_pos[t0 + c + tt];   // float32 product
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const float qo = zr[cq + hd * D + other], ko = zr[ck + hd * D + other];
        qv = lo ? qv * cs - qo * sn : qv * cs + qo * sn;
        kv = lo ? kv * cs - ko * sn : kv * cs + ko * sn;
      }
      qk[e] = make_float2(qv, kv * k_scale);
    }
    for (int e = threadIdx.x; e < cn * cw; e += blockDim.x) {
      const int tt = e / cw, jj = e - tt * cw;
      const float* zr = z + (size_t)(t0 + c + tt) * ld;
      sv[tt * CW + jj] = zr[cv + hd * DV + c0 + jj];
      sg[tt * CW + jj] = zr[cg + hd * DV + c0 + jj];
    }
    __syncthreads();
    if (own) {
      for (int tt = 0; tt < cn; ++tt) {
        const float vj = sv[tt * CW + j];
        const float2* x = qk + tt * D;
        float num = 0.f;
        if (R > 0) {
          float n4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int q = 0; q < (R > 0 ? R : 1); ++q) {
            const float2 xi = x[i0 + q];      // no branch, as in wkv_scan_kernel
            const float s = fmaf(a, Sr[q], xi.y * vj);
            Sr[q] = s;
            const float with = fmaf(s, xi.x, n4[q & 3]);
            n4[q & 3] = q < cnt ? with : n4[q & 3];
          }
          num = (n4[0] + n4[1]) + (n4[2] + n4[3]);
        } else {
          for (int ib = i0; ib < i0 + cnt; ib += 8) {   // eight rows at a time, as in wkv_scan_kernel
            float2 xi[8];
            float sc[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int i = min(ib + q, i0 + cnt - 1);
              xi[q] = x[i];
              sc[q] = S[i * CW + j];
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              if (ib + q < i0 + cnt) {
                const float s = fmaf(a, sc[q], xi[q].y * vj);
                S[(ib + q) * CW + j] = s;
                num = fmaf(s, xi[q].x, num);
              }
            }
          }
        }
        snum[(tt * P + part) * CW + j] = num;
      }
    }
    __syncthreads();
    if (raw != nullptr) {
      for (int e = threadIdx.x; e < cn * cw; e += blockDim.x) {
        const int tt = e / cw, jj = e - tt * cw;
        float num = 0.f;
        for (int pp = 0; pp < P; ++pp) num += snum[(tt * P + pp) * CW + jj];
        raw[(size_t)(t0 + c + tt) * H * DV + hd * DV + c0 + jj] = num;
      }
    } else {
      // one slice: the head's unit norm and the gate here, a warp a token
      for (int tt = warp; tt < cn; tt += warps) {
        float nv[8];   // value rows of up to 256 a lane's eight; beyond, the sums are formed again
        float ss = 0.f;
        for (int i = lane, q = 0; i < DV; i += 32, ++q) {
          float num = 0.f;
          for (int pp = 0; pp < P; ++pp) num += snum[(tt * P + pp) * CW + i];
          if (q < 8) nv[q] = num;
          ss = fmaf(num, num, ss);
        }
        const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)DV + eps);
        T* orow = out + (size_t)(t0 + c + tt) * H * DV + hd * DV;
        for (int i = lane, q = 0; i < DV; i += 32, ++q) {
          float num = 0.f;
          if (q < 8) {
            num = nv[q];
          } else {
            for (int pp = 0; pp < P; ++pp) num += snum[(tt * P + pp) * CW + i];
          }
          const float gi = sg[tt * CW + i];
          orow[i] = from_f32<T>(num * inv * (gi / (1.0f + expf(-gi))));
        }
      }
    }
    __syncthreads();
  }
  if (R > 0) {
#pragma unroll
    for (int q = 0; q < (R > 0 ? R : 1); ++q)
      if (own && q < cnt) Sg[(size_t)(i0 + q) * DV + j] = Sr[q];
  } else {
    for (int e = threadIdx.x; e < D * cw; e += blockDim.x) {
      const int i = e / cw, jj = e - i * cw;
      Sg[(size_t)i * DV + jj] = S[i * CW + jj];
    }
  }
}

static size_t retention_smem_bytes(int D, int CW, int P, int R) {
  const size_t state = R ? 0 : (size_t)((D * CW + 3) & ~3);
  return (state + (size_t)SCAN_CT * (2 * D + (2 + P) * CW) + 64 * 2) * sizeof(float);
}

// `decay`: float32 [H] on the device. `inv_freq`: float32 [rot_dim / 2] (may be null when
// rot_dim is 0). `raw`: float32 [T, H * DV] of scratch, as in mb_wkv_scan.
MB_EXPORT int mb_retention_scan(const float* z, int ld, int cq, int ck, int cv, int cg,
                                const float* decay, float k_scale, const float* inv_freq,
                                int rot_dim, const int* tok_pos, float eps, float* state,
                                long long state_stride, long long state_off,
                                const int* seq_start, const int* seq_slot, void* out, float* raw,
                                int dtype, int T_, int B, int H, int D, int DV, void* stream) {
  if (B <= 0) return 0;
  if (D <= 0 || DV <= 0 || D > 512 || DV > 512)
    MB_FAIL("mb_retention_scan: heads of %d x %d values (at most 512 each)", D, DV);
  if (rot_dim < 0 || rot_dim > D || (rot_dim & 1) || (rot_dim > 0 && inv_freq == nullptr))
    MB_FAIL("mb_retention_scan: %d of %d values rotate", rot_dim, D);
  int NS = raw ? scan_slices(B, H, D, DV, 32) : 1, CW, P, R;
  size_t smem;
  for (;; NS *= 2) {
    CW = (DV + NS - 1) / NS;
    P = scan_parts(CW);
    const int per = (D + P - 1) / P;
    R = per <= 8 ? 8 : per <= 16 ? 16 : per <= 32 ? 32 : 0;
    smem = retention_smem_bytes(D, CW, P, R);
    // a head whose state does not fit one block's shared memory: narrower slices of its columns
    if (smem <= 200 * 1024 || !raw || CW <= 32) break;
  }
  if (smem > 200 * 1024)
    MB_FAIL("mb_retention_scan: heads of %d x %d values (what a block stages must fit 200 KB)",
            D, DV);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = (CW + 31) / 32 * 32 * P;
  float* raw_used = NS > 1 ? raw : nullptr;
#define GO(T_t, R_)                                                                            \
  {                                                                                            \
    static size_t configured = 48 * 1024;                                                      \
    if (smem > configured) {                                                                   \
      cudaFuncSetAttribute(retention_scan_kernel<T_t, R_>,                                     \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
      configured = 200 * 1024;                                                                 \
    }                                                                                          \
    mb_launch(retention_scan_kernel<T_t, R_>, dim3(B, H, NS), dim3(threads), smem, s, z, ld,   \
              cq, ck, cv, cg, decay, k_scale, inv_freq, rot_dim, tok_pos, eps, state,          \
              (size_t)state_stride, (size_t)state_off, seq_start, seq_slot, (T_t*)out,         \
              raw_used, H, D, DV);                                                             \
    if (NS > 1) launch_head_norm<T_t>(raw, z + cg, ld, nullptr, eps, 0, out, T_, H, DV, s);    \
  }
#define GOR(T_t)                                                                               \
  switch (R) {                                                                                 \
    case 8: GO(T_t, 8) break;                                                                  \
    case 16: GO(T_t, 16) break;                                                                \
    case 32: GO(T_t, 32) break;                                                                \
    default: GO(T_t, 0)                                                                        \
  }
  if (dtype == MB_F32) GOR(float) else GOR(__nv_bfloat16)
#undef GOR
#undef GO
  MB_CHECK_LAUNCH("mb_retention_scan");
}

// ------------------------------------------------------------------ retention, chunk by chunk
// The same recurrence for a step that brings many tokens of a sequence. The step's tokens of a
// sequence are cut into chunks of C; with n a chunk's tokens, S0 the state before it, g the
// head's decay and t, s counting inside the chunk:
//   o_t = g^(t+1) S0^T q_t + sum_{s <= t} g^(t-s) (q_t . k_s) v_s
//   S_n = g^n S0 + sum_s g^(n-1-s) k_s v_s^T
// Three kernels. (1) Every chunk's own sum U = sum_s g^(n-1-s) k_s v_s^T, all chunks side by
// side. (2) The walk S0(c+1) = g^n S0(c) + U(c) over a sequence's chunks, element by element;
// it leaves S0(c) where U(c) was and the last state in the slot. (3) Every chunk's outputs,
// side by side again: the scores' lower triangle with its decays, both sums, the head's unit
// norm and the gate. All of it float32 on the CUDA cores (scores and state are 32-bit
// quantities); what is gained over the walk token by token is that the chunks of one prompt
// fill the device instead of a block per head. W: float32 [chunks][H][D][DVp], DVp = DV rounded
// up to 4; chunk g of the step belongs to sequence b, chunk c, in the order of the sequences.
__device__ __forceinline__ bool chunk_of(const int* __restrict__ seq_start, int B, int C, int g,
                                         int* b_out, int* c_out) {
  int before = 0;
  for (int b = 0; b < B; ++b) {
    const int nc = (seq_start[b + 1] - seq_start[b] + C - 1) / C;
    if (g < before + nc) {
      *b_out = b;
      *c_out = g - before;
      return true;
    }
    before += nc;
  }
  return false;
}

// q and k of head hd, value i, of the token whose row of z is zr, turned by its position
__device__ __forceinline__ float2 turned_qk(const float* __restrict__ zr, int cq, int ck, int hd,
                                            int D, int i, int rot_dim,
                                            const float* __restrict__ inv_freq, int pos) {
  float qv = zr[cq + hd * D + i], kv = zr[ck + hd * D + i];
  if (i < rot_dim) {
    const int half = rot_dim >> 1;
    const bool lo = i < half;
    const int f = lo ? i : i - half, other = lo ? i + half : i - half;
    const float angle = inv_freq[f] * (float)pos;   // float32 product
    float sn, cs;
    sincosf(angle, &sn, &cs);
    const float qo = zr[cq + hd * D + other], ko = zr[ck + hd * D + other];
    qv = lo ? qv * cs - qo * sn : qv * cs + qo * sn;
    kv = lo ? kv * cs - ko * sn : kv * cs + ko * sn;
  }
  return make_float2(qv, kv);
}

// acc[p][q] += a.p * b.q
__device__ __forceinline__ void outer4(float (&acc)[4][4], const float4 a, const float4 b) {
  acc[0][0] = fmaf(a.x, b.x, acc[0][0]); acc[0][1] = fmaf(a.x, b.y, acc[0][1]);
  acc[0][2] = fmaf(a.x, b.z, acc[0][2]); acc[0][3] = fmaf(a.x, b.w, acc[0][3]);
  acc[1][0] = fmaf(a.y, b.x, acc[1][0]); acc[1][1] = fmaf(a.y, b.y, acc[1][1]);
  acc[1][2] = fmaf(a.y, b.z, acc[1][2]); acc[1][3] = fmaf(a.y, b.w, acc[1][3]);
  acc[2][0] = fmaf(a.z, b.x, acc[2][0]); acc[2][1] = fmaf(a.z, b.y, acc[2][1]);
  acc[2][2] = fmaf(a.z, b.z, acc[2][2]); acc[2][3] = fmaf(a.z, b.w, acc[2][3]);
  acc[3][0] = fmaf(a.w, b.x, acc[3][0]); acc[3][1] = fmaf(a.w, b.y, acc[3][1]);
  acc[3][2] = fmaf(a.w, b.z, acc[3][2]); acc[3][3] = fmaf(a.w, b.w, acc[3][3]);
}

template <int C>
__global__ void __launch_bounds__(256)
retention_chunk_sums_kernel(const float* __restrict__ z, int ld, int ck, int cv,
                            const float* __restrict__ decay, float k_scale,
                            const float* __restrict__ inv_freq, int rot_dim,
                            const int* __restrict__ tok_pos, const int* __restrict__ seq_start,
                            int B, float* __restrict__ W, int H, int D, int DV) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) float rc_smem[];
  __shared__ float gp[C + 1];
  int b, c;
  if (!chunk_of(seq_start, B, C, blockIdx.x, &b, &c)) return;
  const int hd = blockIdx.y, Dp = (D + 3) & ~3, DVp = (DV + 3) & ~3;
  float* ks = rc_smem;            // [C][Dp]  g^(n-1-s) k_s, turned and scaled
  float* vs = ks + C * Dp;        // [C][DVp]
  const int t0 = seq_start[b] + c * C, n = min(C, seq_start[b + 1] - t0);
  const double a = (double)decay[hd];
  for (int e = threadIdx.x; e <= C; e += blockDim.x) gp[e] = (float)pow(a, (double)e);
  __syncthreads();
  for (int e = threadIdx.x; e < C * Dp; e += blockDim.x) {
    const int s = e / Dp, i = e - s * Dp;
    float v = 0.f;
    if (s < n && i < D)
      v = turned_qk(z + (size_t)(t0 + s) * ld, ck, ck, hd, D, i, rot_dim, inv_freq,
                    tok_pos[t0 + s]).y * k_scale * gp[n - 1 - s];
    ks[e] = v;
  }
  for (int e = threadIdx.x; e < C * DVp; e += blockDim.x) {
    const int s = e / DVp, j = e - s * DVp;
    vs[e] = (s < n && j < DV) ? z[(size_t)(t0 + s) * ld + cv + hd * DV + j] : 0.f;
  }
  __syncthreads();
  float* Wc = W + ((size_t)blockIdx.x * H + hd) * D * DVp;
  const int TJ = DVp >> 2, tiles = (Dp >> 2) * TJ;
  for (int tile = threadIdx.x; tile < tiles; tile += blockDim.x) {
    const int ti = tile / TJ, tj = tile - ti * TJ;
    float acc[4][4] = {};
    for (int s = 0; s < n; ++s)
      outer4(acc, *(const float4*)(ks + s * Dp + 4 * ti), *(const float4*)(vs + s * DVp + 4 * tj));
#pragma unroll
    for (int p = 0; p < 4; ++p)
      if (4 * ti + p < D)
        *(float4*)(Wc + (size_t)(4 * ti + p) * DVp + 4 * tj) =
            make_float4(acc[p][0], acc[p][1], acc[p][2], acc[p][3]);
  }
}

template <int C>
__global__ void __launch_bounds__(256)
retention_chunk_carry_kernel(float* __restrict__ W, const float* __restrict__ decay,
                             float* __restrict__ state, size_t state_stride, size_t state_off,
                             const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                             int H, int D, int DV) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int b = blockIdx.z, hd = blockIdx.y, DVp = (DV + 3) & ~3, TJ = DVp >> 2;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= D * TJ) return;
  const int i = e / TJ, j = 4 * (e - i * TJ);
  int first = 0;
  for (int bb = 0; bb < b; ++bb) first += (seq_start[bb + 1] - seq_start[bb] + C - 1) / C;
  const int n = seq_start[b + 1] - seq_start[b], nc = (n + C - 1) / C;
  if (nc == 0) return;
  float* Sg = state + (size_t)seq_slot[b] * state_stride + state_off +
              ((size_t)hd * D + i) * DV + j;
  float4 S = make_float4(Sg[0], j + 1 < DV ? Sg[1] : 0.f, j + 2 < DV ? Sg[2] : 0.f,
                         j + 3 < DV ? Sg[3] : 0.f);
  const double a = (double)decay[hd];
  const float whole = (float)pow(a, (double)C), last = (float)pow(a, (double)(n - (nc - 1) * C));
  const size_t pitch = (size_t)H * D * DVp;
  float* w = W + ((size_t)first * H + hd) * D * DVp + (size_t)i * DVp + j;
  // the chunks' sums do not depend on the state: eight loads in flight, then eight steps
  constexpr int AHEAD = 8;
  for (int c0 = 0; c0 < nc; c0 += AHEAD) {
    float4 u[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k)
      u[k] = c0 + k < nc ? *(const float4*)(w + (size_t)(c0 + k) * pitch)
                         : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      if (c0 + k < nc) {
        *(float4*)(w + (size_t)(c0 + k) * pitch) = S;
        const float f = c0 + k == nc - 1 ? last : whole;
        S = make_float4(fmaf(f, S.x, u[k].x), fmaf(f, S.y, u[k].y), fmaf(f, S.z, u[k].z),
                        fmaf(f, S.w, u[k].w));
      }
    }
  }
  Sg[0] = S.x;
  if (j + 1 < DV) Sg[1] = S.y;
  if (j + 2 < DV) Sg[2] = S.z;
  if (j + 3 < DV) Sg[3] = S.w;
}

template <typename T, int C>
__global__ void __launch_bounds__(256)
retention_chunk_out_kernel(const float* __restrict__ z, int ld, int cq, int ck, int cv, int cg,
                           const float* __restrict__ decay, float k_scale,
                           const float* __restrict__ inv_freq, int rot_dim,
                           const int* __restrict__ tok_pos, float eps,
                           const int* __restrict__ seq_start, int B,
                           const float* __restrict__ W, T* __restrict__ out, int H, int D,
                           int DV) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) float rc_smem[];
  __shared__ float gp[C + 1];
  constexpr int CP = C + 4;       // the pitch of rows that hold one value of every token
  int b, c;
  if (!chunk_of(seq_start, B, C, blockIdx.x, &b, &c)) return;
  const int hd = blockIdx.y, DVp = (DV + 3) & ~3;
  float* qT = rc_smem;            // [D][CP]   q_t[i] at i * CP + t
  float* kT = qT + D * CP;        // [D][CP]
  float* AT = kT + D * CP;        // [C][CP]   g^(t-s) q_t . k_s at s * CP + t, zero above t
  float* vs = AT + C * CP;        // [C][DVp]
  float* os = vs + C * DVp;       // [C][DVp]  the outputs before the head's norm
  const int t0 = seq_start[b] + c * C, n = min(C, seq_start[b + 1] - t0);
  const double a = (double)decay[hd];
  for (int e = threadIdx.x; e <= C; e += blockDim.x) gp[e] = (float)pow(a, (double)e);
  for (int e = threadIdx.x; e < C * D; e += blockDim.x) {
    const int s = e / D, i = e - s * D;
    float2 v = make_float2(0.f, 0.f);
    if (s < n) {
      v = turned_qk(z + (size_t)(t0 + s) * ld, cq, ck, hd, D, i, rot_dim, inv_freq,
                    tok_pos[t0 + s]);
      v.y *= k_scale;
    }
    qT[i * CP + s] = v.x;
    kT[i * CP + s] = v.y;
  }
  for (int e = threadIdx.x; e < C * DVp; e += blockDim.x) {
    const int s = e / DVp, j = e - s * DVp;
    vs[e] = (s < n && j < DV) ? z[(size_t)(t0 + s) * ld + cv + hd * DV + j] : 0.f;
  }
  __syncthreads();
  constexpr int TT = C / 4;
  for (int tile = threadIdx.x; tile < TT * TT; tile += blockDim.x) {
    const int tt = tile / TT, ts = tile - tt * TT;
    if (ts > tt || 4 * tt >= n) continue;
    float acc[4][4] = {};
    for (int i = 0; i < D; ++i)
      outer4(acc, *(const float4*)(qT + i * CP + 4 * tt), *(const float4*)(kT + i * CP + 4 * ts));
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float r[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const int far = 4 * (tt - ts) + p - q;
        r[p] = far >= 0 ? acc[p][q] * gp[far] : 0.f;
      }
      *(float4*)(AT + (4 * ts + q) * CP + 4 * tt) = make_float4(r[0], r[1], r[2], r[3]);
    }
  }
  __syncthreads();
  const float* Wc = W + ((size_t)blockIdx.x * H + hd) * D * DVp;
  const int TJ = DVp >> 2;
  for (int tile = threadIdx.x; tile < TT * TJ; tile += blockDim.x) {
    const int tt = tile / TJ, tj = tile - tt * TJ;
    if (4 * tt >= n) continue;
    float acc[4][4] = {};
    for (int i = 0; i < D; ++i)
      outer4(acc, *(const float4*)(qT + i * CP + 4 * tt),
             __ldg((const float4*)(Wc + (size_t)i * DVp + 4 * tj)));
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float f = gp[min(C, 4 * tt + p + 1)];
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[p][q] *= f;
    }
    const int smax = min(4 * tt + 3, n - 1);
    for (int s = 0; s <= smax; ++s)
      outer4(acc, *(const float4*)(AT + s * CP + 4 * tt), *(const float4*)(vs + s * DVp + 4 * tj));
#pragma unroll
    for (int p = 0; p < 4; ++p)
      *(float4*)(os + (4 * tt + p) * DVp + 4 * tj) =
          make_float4(acc[p][0], acc[p][1], acc[p][2], acc[p][3]);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int t = warp; t < n; t += warps) {
    float ss = 0.f;
    for (int j = lane; j < DV; j += 32) ss = fmaf(os[t * DVp + j], os[t * DVp + j], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)DV + eps);
    const float* gr = z + (size_t)(t0 + t) * ld + cg + hd * DV;
    T* orow = out + (size_t)(t0 + t) * H * DV + hd * DV;
    for (int j = lane; j < DV; j += 32) {
      const float gi = gr[j];
      orow[j] = from_f32<T>(os[t * DVp + j] * inv * (gi / (1.0f + expf(-gi))));
    }
  }
}

static size_t retention_chunk_smem(int C, int D, int DV) {
  const int DVp = (DV + 3) & ~3;
  return sizeof(float) * ((size_t)2 * D * (C + 4) + (size_t)C * (C + 4) + (size_t)2 * C * DVp);
}

// The chunk that heads of D x DV values are walked in by mb_retention_chunked: 64, 32, or 0 when
// even 32 tokens of such a head do not fit a block's shared memory (mb_retention_scan then).
MB_EXPORT int mb_retention_chunk(int D, int DV) {
  if (D <= 0 || DV <= 0) return 0;
  if (retention_chunk_smem(64, D, DV) <= 112 * 1024) return 64;    // two blocks a multiprocessor
  if (retention_chunk_smem(32, D, DV) <= 200 * 1024) return 32;
  return 0;
}

// As mb_retention_scan, chunk by chunk. W: float32 scratch of w_chunks * H * D * ((DV + 3) & ~3)
// values, w_chunks at least (T + C - 1) / C + B with C = mb_retention_chunk(D, DV).
MB_EXPORT int mb_retention_chunked(const float* z, int ld, int cq, int ck, int cv, int cg,
                                   const float* decay, float k_scale, const float* inv_freq,
                                   int rot_dim, const int* tok_pos, float eps, float* state,
                                   long long state_stride, long long state_off,
                                   const int* seq_start, const int* seq_slot, void* out,
                                   float* W, int w_chunks, int dtype, int T_, int B, int H,
                                   int D, int DV, void* stream) {
  if (B <= 0 || T_ <= 0) return 0;
  const int C = mb_retention_chunk(D, DV);
  if (C == 0) MB_FAIL("mb_retention_chunked: heads of %d x %d values fit no chunk", D, DV);
  if (rot_dim < 0 || rot_dim > D || (rot_dim & 1) || (rot_dim > 0 && inv_freq == nullptr))
    MB_FAIL("mb_retention_chunked: %d of %d values rotate", rot_dim, D);
  if (((uintptr_t)W & 15) != 0) MB_FAIL("mb_retention_chunked: scratch off a 16-byte boundary");
  cudaStream_t s = (cudaStream_t)stream;
  const int chunks = (T_ + C - 1) / C + B;
  if (w_chunks < chunks)
    MB_FAIL("mb_retention_chunked: scratch of %d chunks, %d needed", w_chunks, chunks);
  const int Dp = (D + 3) & ~3, DVp = (DV + 3) & ~3;
  const size_t smem1 = sizeof(float) * (size_t)C * (Dp + DVp), smem3 = retention_chunk_smem(C, D, DV);
  const dim3 carry((D * (DVp >> 2) + 255) / 256, H, B);
#define GO(T_t, C_)                                                                            \
  {                                                                                            \
    static bool configured = false;                                                            \
    if (!configured) {                                                                         \
      cudaFuncSetAttribute(retention_chunk_sums_kernel<C_>,                                    \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
      cudaFuncSetAttribute(retention_chunk_out_kernel<T_t, C_>,                                \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
      configured = true;                                                                       \
    }                                                                                          \
    mb_launch(retention_chunk_sums_kernel<C_>, dim3(chunks, H), dim3(256), smem1, s, z, ld, ck, \
              cv, decay, k_scale, inv_freq, rot_dim, tok_pos, seq_start, B, W, H, D, DV);      \
    mb_launch(retention_chunk_carry_kernel<C_>, carry, dim3(256), 0, s, W, decay, state,       \
              (size_t)state_stride, (size_t)state_off, seq_start, seq_slot, H, D, DV);         \
    mb_launch(retention_chunk_out_kernel<T_t, C_>, dim3(chunks, H), dim3(256), smem3, s, z, ld, \
              cq, ck, cv, cg, decay, k_scale, inv_freq, rot_dim, tok_pos, eps, seq_start, B,   \
              (const float*)W, (T_t*)out, H, D, DV);                                           \
  }
  if (dtype == MB_F32) {
    if (C == 64) GO(float, 64) else GO(float, 32)
  } else {
    if (C == 64) GO(__nv_bfloat16, 64) else GO(__nv_bfloat16, 32)
  }
#undef GO
  MB_CHECK_LAUNCH("mb_retention_chunked");
}

// ------------------------------------------------------------------ tanh between two products
template <typename T>
__global__ void tanh_kernel(const float* __restrict__ in, int ld_in, T* __restrict__ out,
                            int rows, int cols) {
  mb_grid_wait();
  mb_grid_launch_next();
  const size_t total = (size_t)rows * cols;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols, c = i - r * cols;
    out[i] = from_f32<T>(tanhf(in[r * ld_in + c]));
  }
}

// out [rows, cols] = tanh(in [rows, cols] float32 with a row pitch of ld_in), rounded to the
// activation type.
MB_EXPORT int mb_tanh(const float* in, int ld_in, void* out, int out_dtype, int rows, int cols,
                      void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const long long want = ((long long)rows * cols + 255) / 256;
  const dim3 grid((unsigned)(want < 148 * 8 ? want : 148 * 8));
  if (out_dtype == MB_F32)
    mb_launch(tanh_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, in, ld_in,
              (float*)out, rows, cols);
  else
    mb_launch(tanh_kernel<__nv_bfloat16>, grid, dim3(256), 0, (cudaStream_t)stream, in, ld_in,
              (__nv_bfloat16*)out, rows, cols);
  MB_CHECK_LAUNCH("mb_tanh");
}
