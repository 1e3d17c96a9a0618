// A selective state-space mixer (the "state-space duality" form with a scalar decay per head) over
// ragged batches, with the state of every request kept in slots between steps.
//
// Per token the input projection gives  z (inner) | x (inner) | B (G*N) | C (G*N) | dt (H);  inner = H * P.
//   1. short causal convolution per channel over x|B|C with bias, then silu; the inputs of the last
//      taps-1 tokens of a request are part of its state, so a portion may start anywhere;
//   2. dt = softplus(dt + dt_bias);   per head h (group g = h / (H / G)):
//        S <- exp(-exp(A_log_h) dt) S + dt B_g x_h^T     (S: N x P, float, one per request and head)
//        y_h = S^T C_g + D_h x_h;
//   3. y * silu(z), unit RMS in equal parts of the row (each by its own mean square), times a weight.
// The decay, dt, the state, y and the norm are float; x, B, C arrive in the element type T.
//
// A request's tokens of one step are neighbours in the batch (rows seq_starts[s] .. seq_starts[s+1]),
// its slot is state_slots[s].  Every (request, head) is scanned by exactly one block, token after token.
#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// One block per token; threads over channels.  conv_state: [slots][taps-1][channels] float, oldest first.
template <typename T>
__global__ void __launch_bounds__(256)
conv_silu_kernel(const T* __restrict__ proj, int ld, int off, int channels, int taps, const T* __restrict__ weight,
                 const T* __restrict__ bias, const float* __restrict__ conv_state, const int* __restrict__ seq_of_token,
                 const int* __restrict__ seq_starts, const int* __restrict__ state_slots, T* __restrict__ out) {
  chain_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const int start = seq_starts[seq];
  const int i = t - start;                                    // index of the token inside its portion
  const float* old = conv_state + (size_t)state_slots[seq] * (taps - 1) * channels;
  for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < channels; ch += gridDim.y * blockDim.x) {
    float acc = bias ? Elem<T>::load(bias + ch) : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int r = i - (taps - 1 - j);                        // portion index of the input under tap j
      const float v = r >= 0 ? Elem<T>::load(proj + (size_t)(start + r) * ld + off + ch)
                             : old[(size_t)(taps - 1 + r) * channels + ch];
      acc = fmaf(Elem<T>::load(weight + (size_t)ch * taps + j), v, acc);
    }
    Elem<T>::store(out + (size_t)t * channels + ch, silu_f(acc));
  }
}

// One block per request: the last taps-1 inputs of (old state, then the portion) become the state.
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const T* __restrict__ proj, int ld, int off, int channels, int taps, float* __restrict__ conv_state,
                         const int* __restrict__ seq_starts, const int* __restrict__ state_slots) {
  chain_wait();
  const int seq = blockIdx.x;
  const int start = seq_starts[seq], n = seq_starts[seq + 1] - start;
  const int K = taps - 1;
  float* st = conv_state + (size_t)state_slots[seq] * K * channels;
  for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < channels; ch += gridDim.y * blockDim.x) {
    for (int k = 0; k < K; ++k) {                             // rising k: entry k + n is read before it is written
      const int src = k + n;
      st[(size_t)k * channels + ch] = src < K ? st[(size_t)src * channels + ch]
                                              : Elem<T>::load(proj + (size_t)(start + src - K) * ld + off + ch);
    }
  }
}

constexpr int kScanChunk = 16;     // tokens staged in shared memory at a time

// One block per (head, request); thread (l, p): column p of the state, rows l * NL .. l * NL + NL - 1, in
// registers.  A chunk of tokens is staged (B, C, x, dt, decay as floats), scanned without a barrier (every
// thread leaves its partial y per token in shared memory), then the L partial sums of a column are added in order.
template <typename T, int NLMAX>
__global__ void __launch_bounds__(512)
ssm_scan_kernel(const T* __restrict__ xbc, int channels, const T* __restrict__ proj, int ld, int off_dt,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ state, const int* __restrict__ seq_starts, const int* __restrict__ state_slots,
                float* __restrict__ y, int H, int P, int N, int G, int L, int NL) {
  chain_wait();
  extern __shared__ float smem[];
  float* b_s = smem;                                   // [chunk][N]
  float* c_s = b_s + kScanChunk * N;                   // [chunk][N]
  float* x_s = c_s + kScanChunk * N;                   // [chunk][P]
  float* dt_s = x_s + kScanChunk * P;                  // [chunk]
  float* decay_s = dt_s + kScanChunk;                  // [chunk]
  float* part_s = decay_s + kScanChunk;                // [chunk][L][P]
  const int h = blockIdx.x, seq = blockIdx.y;
  const int g = h / (H / G);
  const int inner = H * P;
  const int p = threadIdx.x % P, l = threadIdx.x / P;
  const int n0 = l * NL;
  const int start = seq_starts[seq], n_tok = seq_starts[seq + 1] - start;
  float* s_glob = state + (((size_t)state_slots[seq] * H + h) * N) * P;
  float S[NLMAX];
#pragma unroll
  for (int i = 0; i < NLMAX; ++i) S[i] = (i < NL && n0 + i < N) ? s_glob[(size_t)(n0 + i) * P + p] : 0.f;
  const float a = -expf(a_log[h]), bias = dt_bias[h], dskip = d_skip[h];
  for (int c0 = 0; c0 < n_tok; c0 += kScanChunk) {
    const int nc = min(kScanChunk, n_tok - c0);
    __syncthreads();                                   // (the chunk before has been read)
    for (int idx = threadIdx.x; idx < nc * N; idx += blockDim.x) {
      const int k = idx / N, n = idx % N;
      const T* row = xbc + (size_t)(start + c0 + k) * channels;
      b_s[idx] = Elem<T>::load(row + inner + g * N + n);
      c_s[idx] = Elem<T>::load(row + inner + G * N + g * N + n);
    }
    for (int idx = threadIdx.x; idx < nc * P; idx += blockDim.x) {
      const int k = idx / P, pp = idx % P;
      x_s[idx] = Elem<T>::load(xbc + (size_t)(start + c0 + k) * channels + h * P + pp);
    }
    for (int k = threadIdx.x; k < nc; k += blockDim.x) {
      const float dt = softplus_f(Elem<T>::load(proj + (size_t)(start + c0 + k) * ld + off_dt + h) + bias);
      dt_s[k] = dt;
      decay_s[k] = expf(a * dt);
    }
    __syncthreads();
    for (int k = 0; k < nc; ++k) {
      const float decay = decay_s[k], dx = dt_s[k] * x_s[k * P + p];
      const float* bk = b_s + k * N + n0;
      const float* ck = c_s + k * N + n0;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < NLMAX; ++i) {
        if (i < NL && n0 + i < N) {
          S[i] = fmaf(decay, S[i], bk[i] * dx);
          sum = fmaf(S[i], ck[i], sum);
        }
      }
      part_s[(k * L + l) * P + p] = sum;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nc * P; idx += blockDim.x) {
      const int k = idx / P, pp = idx % P;
      float sum = 0.f;
      for (int ll = 0; ll < L; ++ll) sum += part_s[(k * L + ll) * P + pp];
      y[(size_t)(start + c0 + k) * inner + h * P + pp] = sum + dskip * x_s[idx];
    }
  }
#pragma unroll
  for (int i = 0; i < NLMAX; ++i)
    if (i < NL && n0 + i < N) s_glob[(size_t)(n0 + i) * P + p] = S[i];
}

// The same scan for states whose row count is a multiple of NL (8 or 16): a block owns PB (16 or 32) columns of
// one head's state, thread (l, p) rows NL l .. NL l + NL - 1 of column p, so a head gives P / PB blocks of
// N / NL * PB light threads (more warps in flight to hide the dependent steps of a token, and a warp reads B and C
// as 16-byte broadcasts).  Same arithmetic per state entry; the partial sums of a column are added in the order of l.
template <typename T, int NL>
__global__ void __launch_bounds__(512)
ssm_scan16_kernel(const T* __restrict__ xbc, int channels, const T* __restrict__ proj, int ld, int off_dt,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                  float* __restrict__ state, const int* __restrict__ seq_starts, const int* __restrict__ state_slots,
                  float* __restrict__ y, int H, int P, int N, int G, int PB) {
  chain_wait();
  extern __shared__ __align__(16) float smem[];
  const int L = N / NL;
  float* b_s = smem;                                   // [chunk][N]
  float* c_s = b_s + kScanChunk * N;                   // [chunk][N]
  float* x_s = c_s + kScanChunk * N;                   // [chunk][PB]
  float* dt_s = x_s + kScanChunk * PB;                 // [chunk]
  float* decay_s = dt_s + kScanChunk;                  // [chunk]
  float* part_s = decay_s + kScanChunk;                // [chunk][L][PB]
  const int h = blockIdx.x, seq = blockIdx.y, p0 = blockIdx.z * PB;
  const int g = h / (H / G);
  const int inner = H * P;
  const int p = threadIdx.x % PB, l = threadIdx.x / PB;
  const int n0 = l * NL;
  const int start = seq_starts[seq], n_tok = seq_starts[seq + 1] - start;
  float* s_glob = state + (((size_t)state_slots[seq] * H + h) * N + n0) * P + p0 + p;
  float S[NL];
#pragma unroll
  for (int i = 0; i < NL; ++i) S[i] = s_glob[(size_t)i * P];
  const float a = -expf(a_log[h]), bias = dt_bias[h], dskip = d_skip[h];
  for (int c0 = 0; c0 < n_tok; c0 += kScanChunk) {
    const int nc = min(kScanChunk, n_tok - c0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nc * N; idx += blockDim.x) {
      const int k = idx / N, n = idx % N;
      const T* row = xbc + (size_t)(start + c0 + k) * channels;
      b_s[idx] = Elem<T>::load(row + inner + g * N + n);
      c_s[idx] = Elem<T>::load(row + inner + G * N + g * N + n);
    }
    for (int idx = threadIdx.x; idx < nc * PB; idx += blockDim.x) {
      const int k = idx / PB, pp = idx % PB;
      x_s[idx] = Elem<T>::load(xbc + (size_t)(start + c0 + k) * channels + h * P + p0 + pp);
    }
    for (int k = threadIdx.x; k < nc; k += blockDim.x) {
      const float dt = softplus_f(Elem<T>::load(proj + (size_t)(start + c0 + k) * ld + off_dt + h) + bias);
      dt_s[k] = dt;
      decay_s[k] = expf(a * dt);
    }
    __syncthreads();
    for (int k = 0; k < nc; ++k) {
      const float decay = decay_s[k], dx = dt_s[k] * x_s[k * PB + p];
      const float4* bk = reinterpret_cast<const float4*>(b_s + k * N + n0);
      const float4* ck = reinterpret_cast<const float4*>(c_s + k * N + n0);
      float sum = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < NL / 4; ++i4) {
        const float4 b = bk[i4], c = ck[i4];
        S[4 * i4] = fmaf(decay, S[4 * i4], b.x * dx);         sum = fmaf(S[4 * i4], c.x, sum);
        S[4 * i4 + 1] = fmaf(decay, S[4 * i4 + 1], b.y * dx); sum = fmaf(S[4 * i4 + 1], c.y, sum);
        S[4 * i4 + 2] = fmaf(decay, S[4 * i4 + 2], b.z * dx); sum = fmaf(S[4 * i4 + 2], c.z, sum);
        S[4 * i4 + 3] = fmaf(decay, S[4 * i4 + 3], b.w * dx); sum = fmaf(S[4 * i4 + 3], c.w, sum);
      }
      part_s[(k * L + l) * PB + p] = sum;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nc * PB; idx += blockDim.x) {
      const int k = idx / PB, pp = idx % PB;
      float sum = 0.f;
      for (int ll = 0; ll < L; ++ll) sum += part_s[(k * L + ll) * PB + pp];
      y[(size_t)(start + c0 + k) * inner + h * P + p0 + pp] = sum + dskip * x_s[idx];
    }
  }
#pragma unroll
  for (int i = 0; i < NL; ++i) s_glob[(size_t)i * P] = S[i];
}

// One block per (token, part): out = unit_rms(y * silu(z)) * weight over the part's entries.  `gate` may
// be null (no gate), `x` is float (X32) or T.
template <typename T, bool X32>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const void* __restrict__ x_, int x_ld, const T* __restrict__ gate, int gate_ld,
                        const float* __restrict__ weight, T* __restrict__ out, int out_ld, int width, int parts, float eps) {
  chain_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x, part = blockIdx.y;
  const int per = width / parts, lo = part * per;
  float ss = 0.f;
  auto value = [&](int i) {
    float v = X32 ? static_cast<const float*>(x_)[(size_t)t * x_ld + i] : Elem<T>::load(static_cast<const T*>(x_) + (size_t)t * x_ld + i);
    if (gate) v *= silu_f(Elem<T>::load(gate + (size_t)t * gate_ld + i));
    return v;
  };
  for (int i = lo + threadIdx.x; i < lo + per; i += blockDim.x) {
    const float v = value(i);
    ss += v * v;
  }
  const float rs = rsqrtf(block_sum(ss, scratch) / (float)per + eps);
  for (int i = lo + threadIdx.x; i < lo + per; i += blockDim.x)
    Elem<T>::store(out + (size_t)t * out_ld + i, value(i) * rs * weight[i]);
}

}  // namespace

ERB_EXPORT int erb_conv_silu(const void* proj, int n_tokens, int ld, int off, int channels, int taps, const void* weight,
                             const void* bias, const float* conv_state, const int* seq_of_token, const int* seq_starts,
                             const int* state_slots, void* out, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (channels <= 0 || taps < 1 || (taps > 1 && !conv_state)) return fail(ERB_ERR_ARG, "conv_silu: bad sizes");
  launch_chained(conv_silu_kernel<elem_t>, dim3(n_tokens, n_tokens < 64 ? (channels + 255) / 256 : 1), dim3(256), 0, (cudaStream_t)stream, (const elem_t*)proj, ld, off,
                 channels, taps, (const elem_t*)weight, (const elem_t*)bias, conv_state, seq_of_token, seq_starts, state_slots,
                 (elem_t*)out);
  return check_launch("conv_silu");
}

ERB_EXPORT int erb_conv_state_update(const void* proj, int n_seqs, int ld, int off, int channels, int taps, float* conv_state,
                                     const int* seq_starts, const int* state_slots, void* stream) {
  if (n_seqs <= 0 || taps <= 1) return ERB_OK;
  launch_chained(conv_state_update_kernel<elem_t>, dim3(n_seqs, (channels + 255) / 256), dim3(256), 0, (cudaStream_t)stream, (const elem_t*)proj, ld,
                 off, channels, taps, conv_state, seq_starts, state_slots);
  return check_launch("conv_state_update");
}

ERB_EXPORT int erb_ssm_scan(const void* xbc, int channels, const void* proj, int ld, int off_dt, const float* dt_bias,
                            const float* a_log, const float* d_skip, float* state, const int* seq_starts,
                            const int* state_slots, float* y, int n_seqs, int n_tokens, int H, int P, int N, int G, void* stream) {
  if (n_seqs <= 0) return ERB_OK;
  if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G || P > 512) return fail(ERB_ERR_ARG, "ssm_scan: bad sizes (columns of at most 512)");
  const int PB = P % 32 == 0 ? 32 : (P % 16 == 0 ? 16 : 0);
  // rows per thread: 16 for a step of single tokens (fewer, busier threads: the step is the state's read and write),
  // 8 where portions are walked and that still gives a block of at most 512 threads (twice the warps to hide a token's
  // dependent steps).  The two differ in the order in which a column's partial sums are added, that is by rounding.
  const int NLc = (n_tokens > n_seqs && N % 8 == 0 && (N / 8) * PB <= 512) ? 8 : 16;
  if (PB && N % NLc == 0 && (N / NLc) * PB <= 512) {
    const int L = N / NLc;
    const size_t smem16 = sizeof(float) * ((size_t)kScanChunk * (2 * N + PB + 2 + (size_t)L * PB));
    auto kern = NLc == 8 ? ssm_scan16_kernel<elem_t, 8> : ssm_scan16_kernel<elem_t, 16>;
    if (smem16 > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem16);
      if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "ssm_scan: %s", cudaGetErrorString(e));
    }
    launch_chained(kern, dim3(H, n_seqs, P / PB), dim3(L * PB), smem16, (cudaStream_t)stream,
                   (const elem_t*)xbc, channels, (const elem_t*)proj, ld, off_dt, dt_bias, a_log, d_skip, state, seq_starts,
                   state_slots, y, H, P, N, G, PB);
    return check_launch("ssm_scan");
  }
  int L = 512 / P;                       // threads that share a column of the state
  if (L > 4) L = 4;
  if (L > N) L = N;
  int NL = (N + L - 1) / L;
  if (NL > 64) return fail(ERB_ERR_UNSUPPORTED, "ssm_scan: a state of %d rows with columns of %d (at most %d rows)", N, P, 64 * L);
  const size_t smem = sizeof(float) * ((size_t)kScanChunk * (2 * N + P + 2 + (size_t)L * P));
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "ssm_scan: sizes need %zu bytes of shared memory", smem);
  auto kernel = NL <= 16 ? ssm_scan_kernel<elem_t, 16> : ssm_scan_kernel<elem_t, 64>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "ssm_scan: %s", cudaGetErrorString(e));
  }
  launch_chained(kernel, dim3(H, n_seqs), dim3(L * P), smem, (cudaStream_t)stream, (const elem_t*)xbc, channels,
                 (const elem_t*)proj, ld, off_dt, dt_bias, a_log, d_skip, state, seq_starts, state_slots, y, H, P, N, G, L, NL);
  return check_launch("ssm_scan");
}

ERB_EXPORT int erb_gated_group_norm(const void* x, int x_is_float, int x_ld, const void* gate, int gate_ld, const float* weight,
                                    void* out, int out_ld, int n_tokens, int width, int parts, float eps, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (width <= 0 || parts <= 0 || width % parts) return fail(ERB_ERR_ARG, "gated_group_norm: the parts must divide the width");
  if (x_is_float)
    launch_chained(gated_group_norm_kernel<elem_t, true>, dim3(n_tokens, parts), dim3(256), 0, (cudaStream_t)stream, x, x_ld,
                   (const elem_t*)gate, gate_ld, weight, (elem_t*)out, out_ld, width, parts, eps);
  else
    launch_chained(gated_group_norm_kernel<elem_t, false>, dim3(n_tokens, parts), dim3(256), 0, (cudaStream_t)stream, x, x_ld,
                   (const elem_t*)gate, gate_ld, weight, (elem_t*)out, out_ld, width, parts, eps);
  return check_launch("gated_group_norm");
}
