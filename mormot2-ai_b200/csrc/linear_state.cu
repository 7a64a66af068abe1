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
// owns rows of ONE column in registers: P neighbouring lanes share a column's D rows (eight
// each), their partial dot products meet by shuffles, and nothing else is
// exchanged between threads inside a token. A block has a slice of a head's columns; up to 32
// tokens are staged in shared memory at a time, the next chunk's copies under way while one
// is walked, and a chunk is walked without a barrier.
//
//   short_conv   y_t = silu(sum_j w[c, j] x_(t - taps + 1 + j)) per channel, the inputs before
//                a step's first token from the state (zeros at a sequence's start)
#include "common.cuh"

MB_DEFINE_LAST_ERROR


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
  int H, D, DV, P, CW, CT;
};

__device__ __forceinline__ void ls_copy4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void ls_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void ls_wait_but_one() {
  asm volatile("cp.async.wait_group 1;" ::: "memory");
}

// Shared memory: two buffers, each [q | k | decay logits (mode 0)] of CT tokens x DP values and
// CT x CW values of v; then CT x CW outputs and four numbers a token. A token's D values of
// q, k and the decays lie in P parts of R + 4 places (R used): part p is what lane p of a
// column reads, sixteen bytes at a time, and the four places of padding keep the parts of a
// warp on different banks. While a chunk is walked the next one's values are already on their
// way (asynchronous copies of four bytes, whatever the alignment of the rows).
template <typename T, int MODE, int R>
__global__ void __launch_bounds__(512, 1) linear_state_scan_kernel(const LsArgs a) {
  mb_grid_wait();
  mb_grid_launch_next();
  extern __shared__ __align__(16) float ls_smem[];
  constexpr int RP = R + 4, NV = MODE == 0 ? 3 : 2;
  const int D = a.D, DV = a.DV, P = a.P, CW = a.CW, CT = a.CT, DP = P * RP;
  const int BUF = NV * CT * DP + CT * CW;
  float* so = ls_smem + 2 * BUF;              // [CT][CW]
  float* sc = so + CT * CW;                   // [2][CT][8]: decay, beta, factor of q, factor of k,
                                              // k . q; places 6 and 7 receive the two logits
  const int b = blockIdx.x, hd = blockIdx.y, g = hd / a.group;
  const int c0 = blockIdx.z * CW, cw = max(0, min(DV, c0 + CW) - c0);
  const int j = threadIdx.x / P, p = threadIdx.x - j * P;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t0 = a.seq_start[b], n = a.seq_start[b + 1] - t0;
  float* Sg = a.state + (size_t)a.seq_slot[b] * a.state_stride + a.state_off +
              (size_t)hd * D * DV + c0;
  const bool own = j < cw;
  // the places that no copy writes (padding, rows behind D, columns behind cw) stay zero
  for (int e = threadIdx.x; e < 2 * BUF; e += blockDim.x) ls_smem[e] = 0.f;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = p * R + r;
    S[r] = (own && i < D) ? Sg[(size_t)i * DV + j] : 0.f;
  }
  __syncthreads();
  const float q_scale = rsqrtf((float)D);
  const int chunks = (n + CT - 1) / CT;

  auto issue = [&](int ci) {      // chunk ci into buffer ci & 1
    if (ci < chunks) {
      float* qb = ls_smem + (ci & 1) * BUF;
      float* kb = qb + CT * DP;
      float* ab = kb + CT * DP;
      float* vb = qb + NV * CT * DP;
      const int cn = min(CT, n - ci * CT);
      for (int tt = warp; tt < cn; tt += warps) {       // a warp a token, a value a lane
        const size_t row = (size_t)(t0 + ci * CT + tt);
        const float* qr = a.qkv + row * a.ldq + a.cq + g * D;
        const float* kr = a.qkv + row * a.ldq + a.ck + g * D;
        const float* ar = MODE == 0 ? a.za + row * a.lda + a.ca + hd * D : nullptr;
        for (int i = lane; i < D; i += 32) {
          const int dst = tt * DP + (i / R) * RP + (i % R);
          ls_copy4(qb + dst, qr + i);
          ls_copy4(kb + dst, kr + i);
          if (MODE == 0) ls_copy4(ab + dst, ar + i);
        }
        const float* vr = a.qkv + row * a.ldq + a.cv + hd * DV + c0;
        for (int jj = lane; jj < cw; jj += 32) ls_copy4(vb + tt * CW + jj, vr + jj);
        if (MODE == 1 && lane < 2)
          ls_copy4(sc + ((ci & 1) * CT + tt) * 8 + 6 + lane,
                   a.zs + row * a.lds + (lane ? a.cd : a.cb) + hd);
      }
    }
    ls_commit();
  };

  issue(0);
  for (int ci = 0; ci < chunks; ++ci) {
    const int cn = min(CT, n - ci * CT);
    issue(ci + 1);
    ls_wait_but_one();            // chunk ci has landed (this thread's copies)
    __syncthreads();              // ... everyone's
    float* qb = ls_smem + (ci & 1) * BUF;
    float* kb = qb + CT * DP;
    float* ab = kb + CT * DP;
    const float* vb = qb + NV * CT * DP;
    if (MODE == 0) {
      // the decays: sigmoid(z + bias)^(1 / tau), in place
      for (int tt = warp; tt < cn; tt += warps)
        for (int i = lane; i < D; i += 32) {
          const int at = tt * DP + (i / R) * RP + (i % R);
          ab[at] = expf(ls_log_sigmoid(ab[at] + a.abias[hd * D + i]) * a.inv_tau);
        }
    } else {
      // a warp a token: the factors that bring q and k to unit length, the decay and beta
      for (int tt = warp; tt < cn; tt += warps) {
        float ssq = 0.f, ssk = 0.f, dot = 0.f;
        for (int i = lane; i < D; i += 32) {
          const int at = tt * DP + (i / R) * RP + (i % R);
          ssq = fmaf(qb[at], qb[at], ssq);
          ssk = fmaf(kb[at], kb[at], ssk);
          dot = fmaf(kb[at], qb[at], dot);
        }
        ssq = warp_sum(ssq);
        ssk = warp_sum(ssk);
        dot = warp_sum(dot);
        if (lane == 0) {
          float* n8 = sc + ((ci & 1) * CT + tt) * 8;
          const float zb = n8[6], zd = n8[7];
          n8[0] = expf(-expf(a.a_log[hd]) * ls_softplus(zd + a.dt_bias[hd]));
          n8[1] = 1.0f / (1.0f + expf(-zb));
          n8[2] = q_scale / sqrtf(ssq + a.unit_eps);
          n8[3] = 1.0f / sqrtf(ssk + a.unit_eps);
          n8[4] = dot;
        }
      }
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float vj = vb[tt * CW + min(j, CW - 1)];
      const float4* q4 = (const float4*)(qb + tt * DP + p * RP);
      const float4* k4 = (const float4*)(kb + tt * DP + p * RP);
      float o0 = 0.f, o1 = 0.f, o;
      if (MODE == 0) {
        const float4* a4 = (const float4*)(ab + tt * DP + p * RP);
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 al = a4[r >> 2], kk = k4[r >> 2], qq = q4[r >> 2];
          S[r] = fmaf(al.x, S[r], kk.x * vj);
          S[r + 1] = fmaf(al.y, S[r + 1], kk.y * vj);
          S[r + 2] = fmaf(al.z, S[r + 2], kk.z * vj);
          S[r + 3] = fmaf(al.w, S[r + 3], kk.w * vj);
          o0 = fmaf(S[r], qq.x, o0);
          o1 = fmaf(S[r + 1], qq.y, o1);
          o0 = fmaf(S[r + 2], qq.z, o0);
          o1 = fmaf(S[r + 3], qq.w, o1);
        }
        o = (o0 + o1) * q_scale;
      } else {
        // With S' = g S: the read-out (S' + k u^T)^T q = S'^T q + u (k . q), so the sums over the
        // rows of S'^T k and of S'^T q are formed side by side and meet in one round of
        // shuffles; the write into the state is off the path to the output.
        const float* n8 = sc + ((ci & 1) * CT + tt) * 8;
        const float dec = n8[0], beta = n8[1], fq = n8[2], fk = n8[3], kq = n8[4];
        float p0 = 0.f, p1 = 0.f;
        float4 kk[R / 4];
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          kk[r >> 2] = k4[r >> 2];
          const float4 qq = q4[r >> 2];
          S[r] *= dec;
          S[r + 1] *= dec;
          S[r + 2] *= dec;
          S[r + 3] *= dec;
          p0 = fmaf(S[r], kk[r >> 2].x, p0);
          p1 = fmaf(S[r + 1], kk[r >> 2].y, p1);
          p0 = fmaf(S[r + 2], kk[r >> 2].z, p0);
          p1 = fmaf(S[r + 3], kk[r >> 2].w, p1);
          o0 = fmaf(S[r], qq.x, o0);
          o1 = fmaf(S[r + 1], qq.y, o1);
          o0 = fmaf(S[r + 2], qq.z, o0);
          o1 = fmaf(S[r + 3], qq.w, o1);
        }
        float pred = p0 + p1, read = o0 + o1;
        for (int m = 1; m < P; m <<= 1) {
          pred += __shfl_xor_sync(0xffffffffu, pred, m);
          read += __shfl_xor_sync(0xffffffffu, read, m);
        }
        const float uk = beta * (vj - pred * fk) * fk;     // u times the unit key's factor
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          S[r] = fmaf(kk[r >> 2].x, uk, S[r]);
          S[r + 1] = fmaf(kk[r >> 2].y, uk, S[r + 1]);
          S[r + 2] = fmaf(kk[r >> 2].z, uk, S[r + 2]);
          S[r + 3] = fmaf(kk[r >> 2].w, uk, S[r + 3]);
        }
        o = (read + uk * kq) * fq;
      }
      if (MODE == 0)
        for (int m = 1; m < P; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (p == 0 && own) so[tt * CW + j] = o;
    }
    __syncthreads();
    if (a.raw != nullptr) {
      for (int tt = warp; tt < cn; tt += warps) {
        float* rr = a.raw + (size_t)(t0 + ci * CT + tt) * a.H * DV + hd * DV + c0;
        for (int jj = lane; jj < cw; jj += 32) rr[jj] = so[tt * CW + jj];
      }
    } else {
      // one slice: the head's norm, its weight and the gate here, a warp a token
      for (int tt = warp; tt < cn; tt += warps) {
        const size_t row = (size_t)(t0 + ci * CT + tt);
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
    const int i = p * R + r;
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

// how the rows of a column are dealt: P lanes (a power of two, at most 32) with 8 rows each.
// Few rows a lane make many light warps: a warp's time a token is the latency of its chain of
// multiply-adds and shuffles, and several warps a scheduler hide one another's.
#define LS_ROWS 8
static int ls_parts(int D) {
  int p = 1;
  while (p < 32 && p * LS_ROWS < D) p *= 2;
  return p;
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
                                   float* raw, int out_dtype, int T_, int B, int max_new, int H,
                                   int D, int DV, void* stream) {
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
  const int P = ls_parts(D), R = LS_ROWS;
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
  // tokens staged at once: 32, or fewer where a sequence brings fewer (a decode step) or two
  // buffers of them would not fit
  int CT = 32;
  while (CT > 4 && CT / 2 >= max_new) CT /= 2;
  size_t smem = 0;
  for (;; CT /= 2) {
    const size_t buf = (size_t)(mode == 0 ? 3 : 2) * CT * P * (R + 4) + (size_t)CT * CW;
    smem = (2 * buf + (size_t)CT * CW + 16 * CT) * sizeof(float);
    if (smem <= 160 * 1024 || CT == 4) break;
  }
  if (smem > 200 * 1024)
    MB_FAIL("mb_linear_state_scan: heads of %d x %d values need %zu bytes of shared memory", D,
            DV, smem);
  a.CT = CT;
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
#define GOR(T_t, M_) GO(T_t, M_, LS_ROWS)
#define GOM(T_t)                                                                               \
  if (mode == 0) { GOR(T_t, 0) } else { GOR(T_t, 1) }
  if (out_dtype == MB_F32) { GOM(float) } else { GOM(__nv_bfloat16) }
#undef GOM
#undef GOR
#undef GO
  MB_CHECK_LAUNCH("mb_linear_state_scan");
}
