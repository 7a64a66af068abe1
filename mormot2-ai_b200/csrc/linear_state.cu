// Linear-attention mixers whose matrix state per head is decayed and written token by token:
//
//   gated linear attention   S <- diag(a_t) S + k_t v_t^T,  o_t = S^T q_t, with a decay per key
//                            channel a = sigmoid(z + b)^(1/tau) and q scaled by D^(-1/2)
//   gated delta rule         S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;
//                            o_t = S^T q_t, with q and k brought to unit length per head (q also
//                            times D^(-1/2)), beta = sigmoid(.), g = exp(-exp(A) softplus(. + dt))
//
// and, for both, each head's o over its root mean square, times a weight shared by the heads,
// times silu(gate). The state (D x DV float32 per head) lives in the engine's state arena, is
// read when a step begins and written when it ends. Everything here is float32.
//
// A column of the state is independent of every other column in both recurrences, so a thread
// owns rows of ONE column in registers: P neighbouring lanes share a column's D rows (row
// p + P r for r < R), their partial dot products meet by shuffles, and nothing else is
// exchanged between threads inside a token. A block has a slice of a head's columns; sixteen
// tokens are staged in shared memory at a time (q, k and the decays prepared by a warp a
// token), then walked without a barrier.
//
//   short_conv   y_t = silu(sum_j w[c, j] x_(t - taps + 1 + j)) per channel, the inputs before
//                a step's first token from the state (zeros at a sequence's start)
#include "common.cuh"

MB_DEFINE_LAST_ERROR

#define LS_CT 16

__device__ __forceinline__ float ls_log_sigmoid(float x) {
  return fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
}

__device__ __forceinline__ float ls_softplus(float x) {
  return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
}

// ------------------------------------------------------------------ short convolution
// in: float32 [T, ld], channel c at column col0 + c; w: float32 [C, taps], the last tap is the
// current token's; state of a slot: [taps - 1][C] inputs before the step, oldest first.
__global__ void short_conv_kernel(const float* __restrict__ in, int ld, int col0,
                                  const float* __restrict__ w, int taps, int C,
                                  const float* __restrict__ state, size_t state_stride,
                                  size_t state_off, const int* __restrict__ tok_seq,
                                  const int* __restrict__ seq_start,
                                  const int* __restrict__ seq_slot, float* __restrict__ out,
                                  int ldo) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  const int t0 = seq_start[b];
  const float* st = state + (size_t)seq_slot[b] * state_stride + state_off;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int src = t - (taps - 1) + j;
      const float xv = src >= t0 ? in[(size_t)src * ld + col0 + c]
                                 : st[(size_t)(taps - 1 - (t0 - src)) * C + c];
      acc = fmaf(w[(size_t)c * taps + j], xv, acc);
    }
    out[(size_t)t * ldo + c] = acc / (1.0f + expf(-acc));
  }
}

// the state after the step: the last taps - 1 inputs of every sequence (older ones move up)
__global__ void short_conv_state_kernel(const float* __restrict__ in, int ld, int col0, int taps,
                                        int C, float* __restrict__ state, size_t state_stride,
                                        size_t state_off, const int* __restrict__ seq_start,
                                        const int* __restrict__ seq_slot) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int b = blockIdx.x;
  const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
  float* st = state + (size_t)seq_slot[b] * state_stride + state_off;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float keep[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < taps - 1) {
        const int idx = n - (taps - 1) + j;     // the step's row that lands in place j
        keep[j] = idx >= 0 ? in[(size_t)(t0 + idx) * ld + col0 + c] : st[(size_t)(n + j) * C + c];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < taps - 1) st[(size_t)j * C + c] = keep[j];
  }
}

MB_EXPORT int mb_short_conv(const float* in, int ld, int col0, const float* w, int taps, int C,
                            float* state, long long state_stride, long long state_off,
                            const int* tok_seq, const int* seq_start, const int* seq_slot,
                            float* out, int ldo, int T, int B, void* stream) {
  if (T <= 0) return 0;
  if (taps < 1 || taps > 9) MB_FAIL("mb_short_conv: %d taps (1 to 9)", taps);
  cudaStream_t s = (cudaStream_t)stream;
  const int by = (C + 255) / 256;
  mb_launch(short_conv_kernel, dim3(T, by), dim3(256), 0, s, in, ld, col0, w, taps, C,
            (const float*)state, (size_t)state_stride, (size_t)state_off, tok_seq, seq_start,
            seq_slot, out, ldo);
  if (taps > 1)
    mb_launch(short_conv_state_kernel, dim3(B, by), dim3(256), 0, s, in, ld, col0, taps, C, state,
              (size_t)state_stride, (size_t)state_off, seq_start, seq_slot);
  MB_CHECK_LAUNCH("mb_short_conv");
}

// ------------------------------------------------------------------ the walk over the tokens
struct LsArgs {
  const float* qkv;      // q of group g at cq + g * D, k at ck + g * D, v of head h at cv + h * DV
  int ldq, cq, ck, cv, group;   // group: heads that share one q/k group
  // decay per key channel (mode 0): logits za [T, lda] at ca + h * D, bias abias [H * D]
  const float* za;
  int lda, ca;
  const float* abias;
  float inv_tau;
  // scalars per head (mode 1): zs [T, lds], beta's logit at cb + h, the decay's at cd + h
  const float* zs;
  int lds, cb, cd;
  const float* a_log;
  const float* dt_bias;
  float unit_eps;
  // output: gate logits [T, ldg] at cg + h * DV, norm weight [DV], eps
  const float* gate;
  int ldg, cg;
  const float* normw;
  float eps;
  float* state;
  size_t state_stride, state_off;
  const int* seq_start;
  const int* seq_slot;
  void* out;             // [T, H * DV] of the activation type (one slice of columns a head)
  float* raw;            // [T, H * DV] float32 (several slices; normed by a kernel after)
  int H, D, DV, P, CW;
};

template <typename T, int MODE, int R>
__global__ void __launch_bounds__(512, 1) linear_state_scan_kernel(const LsArgs a) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) float ls_smem[];
  const int D = a.D, DV = a.DV, P = a.P, CW = a.CW, Dp = P * R;
  float* sq = ls_smem;                        // [CT][Dp], zeros behind D
  float* sk = sq + LS_CT * Dp;                // [CT][Dp]
  float* sa = sk + LS_CT * Dp;                // [CT][Dp] (mode 0)
  float* sv = sa + (MODE == 0 ? LS_CT * Dp : 0);   // [CT][CW]
  float* so = sv + LS_CT * CW;                // [CT][CW]
  float* sc = so + LS_CT * CW;                // [CT][2]: decay, beta (mode 1)
  const int b = blockIdx.x, hd = blockIdx.y, g = hd / a.group;
  const int c0 = blockIdx.z * CW, cw = max(0, min(DV, c0 + CW) - c0);
  const int j = threadIdx.x / P, p = threadIdx.x - j * P;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t0 = a.seq_start[b], n = a.seq_start[b + 1] - t0;
  float* Sg = a.state + (size_t)a.seq_slot[b] * a.state_stride + a.state_off +
              (size_t)hd * D * DV + c0;
  const bool own = j < cw;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = p + P * r;
    S[r] = (own && i < D) ? Sg[(size_t)i * DV + j] : 0.f;
  }
  const float q_scale = rsqrtf((float)D);
  for (int c = 0; c < n; c += LS_CT) {
    const int cn = min(LS_CT, n - c);
    // a warp a token: q and k (and the decays) as the recurrence takes them
    for (int tt = warp; tt < cn; tt += warps) {
      const size_t row = (size_t)(t0 + c + tt);
      const float* qr = a.qkv + row * a.ldq + a.cq + g * D;
      const float* kr = a.qkv + row * a.ldq + a.ck + g * D;
      float fq = q_scale, fk = 1.f;
      if (MODE == 1) {
        float ssq = 0.f, ssk = 0.f;
        for (int i = lane; i < D; i += 32) {
          ssq = fmaf(qr[i], qr[i], ssq);
          ssk = fmaf(kr[i], kr[i], ssk);
        }
        fq = q_scale / sqrtf(warp_sum(ssq) + a.unit_eps);
        fk = 1.0f / sqrtf(warp_sum(ssk) + a.unit_eps);
        if (lane == 0) {
          const float zb = a.zs[row * a.lds + a.cb + hd], zd = a.zs[row * a.lds + a.cd + hd];
          sc[2 * tt] = expf(-expf(a.a_log[hd]) * ls_softplus(zd + a.dt_bias[hd]));
          sc[2 * tt + 1] = 1.0f / (1.0f + expf(-zb));
        }
      }
      for (int i = lane; i < Dp; i += 32) {
        sq[tt * Dp + i] = i < D ? qr[i] * fq : 0.f;
        sk[tt * Dp + i] = i < D ? kr[i] * fk : 0.f;
        if (MODE == 0)
          sa[tt * Dp + i] = i < D ? expf(ls_log_sigmoid(a.za[row * a.lda + a.ca + hd * D + i] +
                                                        a.abias[hd * D + i]) * a.inv_tau)
                                  : 0.f;
      }
    }
    for (int e = threadIdx.x; e < cn * CW; e += blockDim.x) {
      const int tt = e / CW, jj = e - tt * CW;
      sv[e] = jj < cw ? a.qkv[(size_t)(t0 + c + tt) * a.ldq + a.cv + hd * DV + c0 + jj] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float vj = sv[tt * CW + min(j, CW - 1)];
      const float* q = sq + tt * Dp + p;
      const float* k = sk + tt * Dp + p;
      float o0 = 0.f, o1 = 0.f;
      if (MODE == 0) {
        const float* al = sa + tt * Dp + p;
#pragma unroll
        for (int r = 0; r < R; r += 2) {
          S[r] = fmaf(al[P * r], S[r], k[P * r] * vj);
          o0 = fmaf(S[r], q[P * r], o0);
          S[r + 1] = fmaf(al[P * (r + 1)], S[r + 1], k[P * (r + 1)] * vj);
          o1 = fmaf(S[r + 1], q[P * (r + 1)], o1);
        }
      } else {
        const float dec = sc[2 * tt], beta = sc[2 * tt + 1];
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int r = 0; r < R; r += 2) {
          S[r] *= dec;
          p0 = fmaf(S[r], k[P * r], p0);
          S[r + 1] *= dec;
          p1 = fmaf(S[r + 1], k[P * (r + 1)], p1);
        }
        float pred = p0 + p1;
        for (int m = 1; m < P; m <<= 1) pred += __shfl_xor_sync(0xffffffffu, pred, m);
        const float u = beta * (vj - pred);
#pragma unroll
        for (int r = 0; r < R; r += 2) {
          S[r] = fmaf(k[P * r], u, S[r]);
          o0 = fmaf(S[r], q[P * r], o0);
          S[r + 1] = fmaf(k[P * (r + 1)], u, S[r + 1]);
          o1 = fmaf(S[r + 1], q[P * (r + 1)], o1);
        }
      }
      float o = o0 + o1;
      for (int m = 1; m < P; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (p == 0 && own) so[tt * CW + j] = o;
    }
    __syncthreads();
    if (a.raw != nullptr) {
      for (int e = threadIdx.x; e < cn * cw; e += blockDim.x) {
        const int tt = e / cw, jj = e - tt * cw;
        a.raw[(size_t)(t0 + c + tt) * a.H * DV + hd * DV + c0 + jj] = so[tt * CW + jj];
      }
    } else {
      // one slice: the head's norm, its weight and the gate here, a warp a token
      for (int tt = warp; tt < cn; tt += warps) {
        const size_t row = (size_t)(t0 + c + tt);
        float ss = 0.f;
        for (int i = lane; i < DV; i += 32) ss = fmaf(so[tt * CW + i], so[tt * CW + i], ss);
        const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)DV + a.eps);
        T* orow = (T*)a.out + row * a.H * DV + hd * DV;
        const float* gr = a.gate + row * a.ldg + a.cg + hd * DV;
        for (int i = lane; i < DV; i += 32) {
          const float gi = gr[i];
          orow[i] = from_f32<T>(so[tt * CW + i] * inv * a.normw[i] * (gi / (1.0f + expf(-gi))));
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = p + P * r;
    if (own && i < D) Sg[(size_t)i * DV + j] = S[r];
  }
}

// out[t, hd, :] = o / rms(o) * normw * silu(gate) for every (token, head), a warp each
template <typename T>
__global__ void ls_head_norm_kernel(const float* __restrict__ raw, const float* __restrict__ gate,
                                    int ldg, int cg, const float* __restrict__ normw, float eps,
                                    T* __restrict__ out, int rows, int H, int DV) {
  mb_grid_wait();
  mb_grid_launch_next();
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= rows) return;
  const int t = idx / H, hd = idx - t * H;
  const float* o = raw + (size_t)idx * DV;
  const float* gr = gate + (size_t)t * ldg + cg + hd * DV;
  float ss = 0.f;
  for (int i = lane; i < DV; i += 32) ss = fmaf(o[i], o[i], ss);
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)DV + eps);
  for (int i = lane; i < DV; i += 32) {
    const float gi = gr[i];
    out[(size_t)idx * DV + i] = from_f32<T>(o[i] * inv * normw[i] * (gi / (1.0f + expf(-gi))));
  }
}

// how the rows of a column are dealt: P lanes (a power of two, at most 8) with R rows each
static void ls_shape(int D, int* P, int* R) {
  int p = 1;
  while (p < 8 && (D + p - 1) / p > 16) p *= 2;
  const int per = (D + p - 1) / p;
  *P = p;
  *R = per <= 8 ? 8 : per <= 16 ? 16 : 32;
}

// mode 0: gated linear attention; mode 1: gated delta rule. `raw`: float32 [T, H * DV] of
// scratch, used when a head's columns are dealt over several blocks (a step with few
// (sequence, head) pairs); the choice depends on the step's shape only.
MB_EXPORT int mb_linear_state_scan(int mode, const float* qkv, int ldq, int cq, int ck, int cv,
                                   int group, const float* za, int lda, int ca,
                                   const float* abias, float inv_tau, const float* zs, int lds,
                                   int cb, int cd, const float* a_log, const float* dt_bias,
                                   float unit_eps, const float* gate, int ldg, int cg,
                                   const float* normw, float eps, float* state,
                                   long long state_stride, long long state_off,
                                   const int* seq_start, const int* seq_slot, void* out,
                                   float* raw, int out_dtype, int T_, int B, int H, int D, int DV,
                                   void* stream) {
  if (B <= 0 || T_ <= 0) return 0;
  if (D <= 0 || D > 256 || DV <= 0 || DV > 1024)
    MB_FAIL("mb_linear_state_scan: heads of %d x %d values (at most 256 x 1024)", D, DV);
  if (group <= 0 || H % group) MB_FAIL("mb_linear_state_scan: %d heads in groups of %d", H, group);
  LsArgs a;
  a.qkv = qkv; a.ldq = ldq; a.cq = cq; a.ck = ck; a.cv = cv; a.group = group;
  a.za = za; a.lda = lda; a.ca = ca; a.abias = abias; a.inv_tau = inv_tau;
  a.zs = zs; a.lds = lds; a.cb = cb; a.cd = cd; a.a_log = a_log; a.dt_bias = dt_bias;
  a.unit_eps = unit_eps; a.gate = gate; a.ldg = ldg; a.cg = cg; a.normw = normw; a.eps = eps;
  a.state = state; a.state_stride = (size_t)state_stride; a.state_off = (size_t)state_off;
  a.seq_start = seq_start; a.seq_slot = seq_slot; a.out = out; a.H = H; a.D = D; a.DV = DV;
  int P, R;
  ls_shape(D, &P, &R);
  // a block's slice of the columns: all of them while the step has blocks enough (and they fit
  // a block), else slices of 32 so that a single prompt does not leave the device idle
  int CW = DV;
  if (B * H < 96 && raw != nullptr) CW = 32;
  if (CW > 512 / P) CW = 512 / P;
  if (CW > DV) CW = DV;
  const int NS = (DV + CW - 1) / CW;
  if (NS > 1 && raw == nullptr) MB_FAIL("mb_linear_state_scan: value rows of %d need scratch", DV);
  a.P = P; a.CW = CW; a.raw = NS > 1 ? raw : nullptr;
  const int threads = (CW * P + 31) / 32 * 32;
  const size_t smem = ((size_t)LS_CT * P * R * (mode == 0 ? 3 : 2) + 2 * LS_CT * CW + 2 * LS_CT) *
                      sizeof(float);
  cudaStream_t s = (cudaStream_t)stream;
#define GO(T_t, M_, R_)                                                                        \
  {                                                                                            \
    static size_t configured = 48 * 1024;                                                      \
    if (smem > configured) {                                                                   \
      cudaFuncSetAttribute(linear_state_scan_kernel<T_t, M_, R_>,                              \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
      configured = 200 * 1024;                                                                 \
    }                                                                                          \
    mb_launch(linear_state_scan_kernel<T_t, M_, R_>, dim3(B, H, NS), dim3(threads), smem, s, a); \
    if (NS > 1)                                                                                \
      mb_launch(ls_head_norm_kernel<T_t>, dim3((T_ * H + 3) / 4), dim3(128), 0, s,             \
                (const float*)raw, gate, ldg, cg, normw, eps, (T_t*)out, T_ * H, H, DV);       \
  }
#define GOR(T_t, M_)                                                                           \
  switch (R) {                                                                                 \
    case 8: GO(T_t, M_, 8) break;                                                              \
    case 16: GO(T_t, M_, 16) break;                                                            \
    default: GO(T_t, M_, 32)                                                                   \
  }
#define GOM(T_t)                                                                               \
  if (mode == 0) { GOR(T_t, 0) } else { GOR(T_t, 1) }
  if (out_dtype == MB_F32) { GOM(float) } else { GOM(__nv_bfloat16) }
#undef GOM
#undef GOR
#undef GO
  MB_CHECK_LAUNCH("mb_linear_state_scan");
}
