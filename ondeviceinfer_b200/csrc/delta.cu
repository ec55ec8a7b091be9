// The gated delta rule with one decay per head and key channel, for ragged batches of token runs.
//
// Per sequence and head the state S [d, dv] (fp32, zero at the start) goes through, for each token in order,
//     S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// (the read-out sees the token's own write).  q, k and v come from a short causal convolution per channel
// followed by SiLU; q and k are made unit vectors per head, q also scaled by d^-1/2; beta = sigmoid(b);
// g = exp(-exp(A_log) softplus(a + dt_bias)) per head and key channel.  Everything after the convolutions'
// rounding is fp32.
//
// Kernels (compile with -DODI_DELTA_DIM=<d>, the key size of a head):
//  conv        y[t, c] = silu(sum_j taps[c, j] x[t - K + 1 + j, c]); inputs before the step come from the
//              sequence's convolution state (the last K-1 inputs, zeros at the start);
//  conv_state  the state after the step: the last K-1 inputs of the sequence;
//  prep        per (token, head): unit q (scaled), unit k, decay g as fp32 [tokens, heads, 3, d], and beta;
//  rule        the recurrence: a block per (sequence, head, block of 32 value columns); a column of S is
//              spread over RS neighbouring lanes (8, or a whole warp for wide heads, so that a token's two dot
//              products are a few FMAs and a shuffle tree), each holding d / RS of its rows in registers; the token's
//              q, k, g, v and beta are staged through shared memory 16 (8 for wide heads) tokens at a time, the next
//              chunk being requested into registers while the current one is worked through;
//  out_norm    per (token, head): o / rms(o) (eps inside the root) * weight * sigmoid(gate), rounded to T.
#include "common.cuh"

#ifndef ODI_DELTA_DIM
#error "compile with -DODI_DELTA_DIM=<key size of a head>"
#endif
#define D ODI_DELTA_DIM
#ifdef ODI_DELTA_RS
#define RS ODI_DELTA_RS                                          // a sweep's choice (a power of two up to 32)
#else
// lanes that share a column of S.  Measured on B200 inside whole prompts of 2,048 tokens (us for the mixer):
// key size 64, 16 heads: 8 lanes 881, 32 lanes 1,084; key size 128, 32 heads: 16 lanes 2,200, 32 lanes 1,742.
#define RS (D <= 8 ? 1 : (D <= 16 ? 2 : (D <= 32 ? 4 : (D <= 64 ? 8 : 32))))
#endif
#define RPT ((D + RS - 1) / RS)                                 // rows of S per lane: every RS-th row of its column (neighbouring lanes read
                                                                // neighbouring words of shared memory; rows side by side per lane measured slower)
#define ROW_OK(i) ((RPT * RS == D) || (i) < D)                   // no test where the rows divide evenly
#define CB 32                                                   // value columns per block
#define TCH (D <= 128 ? 16 : 8)                                 // tokens staged at a time
#define NTH (CB * RS)                                           // threads of the recurrence
#define NPRE ((TCH * 3 * D + NTH - 1) / NTH)                    // staged floats of q, k, g per thread and chunk
#define NVPRE ((TCH * CB + NTH - 1) / NTH)                      // staged values per thread and chunk
#define MAX_TAPS 16

struct DeltaArgs {
  const void* proj;       // [n_tokens, ld_proj] in T: q channels, k channels, v channels, then one beta per head
  const float* taps;      // [C, K]
  float* conv_state;      // [slots, K - 1, C]
  void* conv_out;         // [n_tokens, C] in T
  const float* decay_in;  // [n_tokens, ld_decay]: a (heads * d lanes), then the output gate's lanes
  const float* a_log;     // [heads]
  const float* dt_bias;   // [heads * d]
  float* qkg;             // [n_tokens, heads, 3, d]
  float* beta;            // [n_tokens, heads]
  float* state;           // [slots, heads, d, dv]
  float* o;               // [n_tokens, heads * dv]
  const float* norm_w;    // [dv]
  void* out;              // [n_tokens, heads * dv] in T
  const int* cu_q;
  const int* tok_seq;
  const int* slots;
  int n_tokens, n_seqs, ld_proj, ld_decay, heads, kv_heads, dv, taps_n, C;
  float eps, unit_eps;
};

template <typename T>
__device__ __forceinline__ float conv_input(const DeltaArgs& a, int q_begin, int slot, int idx, int c) {
  // input `idx` of the sequence's run in this step; negative indices reach into the convolution state
  if (idx >= 0) return to_f<T>(((const T*)a.proj)[(size_t)(q_begin + idx) * a.ld_proj + c]);
  return a.conv_state[((size_t)slot * (a.taps_n - 1) + (a.taps_n - 1 + idx)) * a.C + c];
}

template <typename T>
__global__ void __launch_bounds__(256)
delta_conv_kernel(DeltaArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int seq = a.tok_seq[t];
  const int q_begin = a.cu_q[seq], slot = a.slots[seq];
  const int li = t - q_begin;
  float acc = 0.f;
  for (int j = 0; j < a.taps_n; ++j)
    acc = fmaf(a.taps[(size_t)c * a.taps_n + j], conv_input<T>(a, q_begin, slot, li - (a.taps_n - 1) + j, c), acc);
  ((T*)a.conv_out)[(size_t)t * a.C + c] = from_f<T>(acc / (1.f + expf(-acc)));
}

template <typename T>
__global__ void __launch_bounds__(256)
delta_conv_state_kernel(DeltaArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin, slot = a.slots[seq];
  const int keep = a.taps_n - 1;
  float next[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j)
    if (j < keep) next[j] = conv_input<T>(a, q_begin, slot, q_len - keep + j, c);
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j)
    if (j < keep) a.conv_state[((size_t)slot * keep + j) * a.C + c] = next[j];
}

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void __launch_bounds__(128)
delta_prep_kernel(DeltaArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x, h = blockIdx.y;
  const int src = h / (a.heads / a.kv_heads);
  const T* y = (const T*)a.conv_out + (size_t)t * a.C;
  const T* q = y + (size_t)src * D;
  const T* k = y + (size_t)a.kv_heads * D + (size_t)src * D;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float qv = to_f<T>(q[i]), kv = to_f<T>(k[i]);
    sq += qv * qv; sk += kv * kv;
  }
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);
  const float qs = 1.0f / sqrtf(sq + a.unit_eps) * (1.0f / sqrtf((float)D));
  const float ks = 1.0f / sqrtf(sk + a.unit_eps);
  const float rate = expf(a.a_log[h]);
  float* dst = a.qkg + ((size_t)t * a.heads + h) * 3 * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    dst[i] = to_f<T>(q[i]) * qs;
    dst[D + i] = to_f<T>(k[i]) * ks;
    const float x = a.decay_in[(size_t)t * a.ld_decay + h * D + i] + a.dt_bias[h * D + i];
    dst[2 * D + i] = expf(-rate * softplus_f(x));
  }
  if (threadIdx.x == 0) {
    const float b = to_f<T>(((const T*)a.proj)[(size_t)t * a.ld_proj + a.C + h]);
    a.beta[(size_t)t * a.heads + h] = 1.f / (1.f + expf(-b));
  }
}

__global__ void __launch_bounds__(CB * RS)
delta_rule_kernel(DeltaArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) float qkg_s[TCH][3 * D];
  __shared__ float v_s[TCH][CB];
  __shared__ float b_s[TCH];
  const int seq = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * CB;
  const int tid = threadIdx.x;
  const int col = tid / RS, rs = tid % RS;
  const int c = c0 + col;
  const bool live = c < a.dv;
  const int q_begin = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_begin, slot = a.slots[seq];
  float* S_g = a.state + ((size_t)slot * a.heads + h) * D * a.dv;
  float S[RPT];
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = rs + RS * ii;
    S[ii] = (live && ROW_OK(i)) ? S_g[(size_t)i * a.dv + c] : 0.f;
  }

  // the chunk that starts at token t0, requested into registers
  float pre[NPRE], vpre[NVPRE], bpre = 0.f;
  auto request = [&](int t0) {
    const int nt = min(TCH, q_len - t0);
#pragma unroll
    for (int j = 0; j < NPRE; ++j) {
      const int i = tid + j * NTH;
      const int tt = i / (3 * D), e = i % (3 * D);
      pre[j] = i < nt * 3 * D ? a.qkg[((size_t)(q_begin + t0 + tt) * a.heads + h) * 3 * D + e] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < NVPRE; ++j) {
      const int i = tid + j * NTH;
      const int tt = i / CB, cc = i % CB;
      vpre[j] = (i < nt * CB && c0 + cc < a.dv) ? a.o[(size_t)(q_begin + t0 + tt) * a.heads * a.dv + h * a.dv + c0 + cc] : 0.f;
    }
    if (tid < nt) bpre = a.beta[(size_t)(q_begin + t0 + tid) * a.heads + h];
  };
  if (q_len > 0) request(0);

  for (int t0 = 0; t0 < q_len; t0 += TCH) {
    const int nt = min(TCH, q_len - t0);
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NPRE; ++j) {
      const int i = tid + j * NTH;
      if (i < TCH * 3 * D) (&qkg_s[0][0])[i] = pre[j];
    }
#pragma unroll
    for (int j = 0; j < NVPRE; ++j) {
      const int i = tid + j * NTH;
      if (i < TCH * CB) (&v_s[0][0])[i] = vpre[j];
    }
    if (tid < TCH) b_s[tid] = bpre;
    __syncthreads();
    if (t0 + TCH < q_len) request(t0 + TCH);      // in flight while this chunk's tokens are worked through
    for (int tt = 0; tt < nt; ++tt) {
      const float* qv = qkg_s[tt];
      const float* kv = qv + D;
      const float* gv = kv + D;
      float dot = 0.f;
#pragma unroll
      for (int ii = 0; ii < RPT; ++ii) {
        const int i = rs + RS * ii;
        if (ROW_OK(i)) { S[ii] *= gv[i]; dot = fmaf(S[ii], kv[i], dot); }
      }
#pragma unroll
      for (int o = RS >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = b_s[tt] * (v_s[tt][col] - dot);
      float out = 0.f;
#pragma unroll
      for (int ii = 0; ii < RPT; ++ii) {
        const int i = rs + RS * ii;
        if (ROW_OK(i)) { S[ii] = fmaf(kv[i], u, S[ii]); out = fmaf(S[ii], qv[i], out); }
      }
#pragma unroll
      for (int o = RS >> 1; o > 0; o >>= 1) out += __shfl_xor_sync(0xffffffffu, out, o);
      // the value of this (token, column) has been read by its only reader: the output takes its place
      if (live && rs == 0) a.o[(size_t)(q_begin + t0 + tt) * a.heads * a.dv + h * a.dv + c] = out;
    }
  }
  if (live) {
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) {
      const int i = rs + RS * ii;
      if (ROW_OK(i)) S_g[(size_t)i * a.dv + c] = S[ii];
    }
  }
}

// Widen the value channels of the convolution output into the fp32 buffer that the rule reads them from and
// then overwrites with its outputs.
template <typename T>
__global__ void delta_values_kernel(DeltaArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int n = a.heads * a.dv;
  const T* v = (const T*)a.conv_out + (size_t)t * a.C + 2 * a.kv_heads * D;
  for (int i = threadIdx.x; i < n; i += blockDim.x) a.o[(size_t)t * n + i] = to_f<T>(v[i]);
}

template <typename T>
__global__ void __launch_bounds__(128)
delta_out_norm_kernel(DeltaArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x, h = blockIdx.y;
  const float* o = a.o + (size_t)t * a.heads * a.dv + h * a.dv;
  const float* gate = a.decay_in + (size_t)t * a.ld_decay + a.heads * D + h * a.dv;
  float ss = 0.f;
  for (int i = threadIdx.x; i < a.dv; i += blockDim.x) ss += o[i] * o[i];
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)a.dv + a.eps);
  T* out = (T*)a.out + (size_t)t * a.heads * a.dv + h * a.dv;
  for (int i = threadIdx.x; i < a.dv; i += blockDim.x)
    out[i] = from_f<T>(o[i] * inv * a.norm_w[i] / (1.f + expf(-gate[i])));
}

extern "C" int odi_delta_dim() { return D; }

// The whole mixer between its input products and its output product: convolutions (and their state), the
// recurrence's inputs, the recurrence, the gated output norm.  Six launches.
extern "C" int odi_delta_rule(const DeltaArgs* args, int dtype, cudaStream_t stream) {
  const DeltaArgs a = *args;
  if (a.n_tokens <= 0 || a.n_seqs <= 0) return 0;
  if (a.taps_n < 1 || a.taps_n > MAX_TAPS || a.heads % a.kv_heads != 0 || a.C != 2 * a.kv_heads * D + a.heads * a.dv)
    return ODI_ERR_ARGUMENT;
  if (a.n_seqs > 65535 || a.heads > 65535) return ODI_ERR_UNSUPPORTED;
  const dim3 cgrid(a.n_tokens, (a.C + 255) / 256), sgrid(a.n_seqs, (a.C + 255) / 256), hgrid(a.n_tokens, a.heads);
  const dim3 rgrid((a.dv + CB - 1) / CB, a.heads, a.n_seqs);
  if (dtype == 0) {
    odi_rc = launch_pdl((delta_conv_kernel<float>), cgrid, dim3(256), 0, stream, a);
    if (a.taps_n > 1) odi_rc = launch_pdl((delta_conv_state_kernel<float>), sgrid, dim3(256), 0, stream, a);
    odi_rc = launch_pdl((delta_prep_kernel<float>), hgrid, dim3(128), 0, stream, a);
    odi_rc = launch_pdl((delta_values_kernel<float>), dim3(a.n_tokens), dim3(128), 0, stream, a);
  } else {
    odi_rc = launch_pdl((delta_conv_kernel<bf16>), cgrid, dim3(256), 0, stream, a);
    if (a.taps_n > 1) odi_rc = launch_pdl((delta_conv_state_kernel<bf16>), sgrid, dim3(256), 0, stream, a);
    odi_rc = launch_pdl((delta_prep_kernel<bf16>), hgrid, dim3(128), 0, stream, a);
    odi_rc = launch_pdl((delta_values_kernel<bf16>), dim3(a.n_tokens), dim3(128), 0, stream, a);
  }
  odi_rc = launch_pdl(delta_rule_kernel, rgrid, dim3(CB * RS), 0, stream, a);
  if (dtype == 0) odi_rc = launch_pdl((delta_out_norm_kernel<float>), hgrid, dim3(128), 0, stream, a);
  else odi_rc = launch_pdl((delta_out_norm_kernel<bf16>), hgrid, dim3(128), 0, stream, a);
  return launch_status();
}
