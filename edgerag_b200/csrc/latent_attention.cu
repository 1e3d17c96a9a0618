// Attention through a latent: per token the cache holds ONE row [c (R) | kr (dr)], the normed
// low-rank latent that every head's keys and values are made from and one rotated key part that all
// heads share.  The heads' up-projections are folded into the queries and the outputs
// ("absorbed"): with  qa_h = W_uk_h^T q_h^unrotated  (R wide)
//     score(h, j) = (qa_h . c_j + q_h^rotated . kr_j) * scale,     o_h = W_uv_h (sum_j p_hj c_j),
// so the kernel is multi-query attention whose key row is the cache row (Dk = R + dr) and whose
// value row is the first R entries of the same row: a key is read once and serves both products and
// every head.  Nothing is up-projected per cached token.
//
// Kernels (all float arithmetic; T is the cache's and the projections' element type):
//   latent_store_kernel      unit-RMS norm of the down-projection's first R entries times a plain weight,
//                            pairwise rotation of its last dr entries, both written to the token's cache
//                            row; optionally the same norm for a query latent.
//   latent_q_rotate_kernel   the rotated part of every head's query, written as float beside the
//                            absorbed part.
//   latent_attention_kernel  one warp per (token, head): online softmax over the visible keys (or over
//                            one split of them), an optional sink in the denominator, an optional
//                            sigmoid gate per head on the result.
//   latent_combine_kernel    merges the splits of a row in split order.
// Rotation convention: neighbouring pairs (2i, 2i+1), angle = position * inv_freq[i] in float.
#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

template <typename T> struct Pair;   // two neighbouring elements as floats
template <> struct Pair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
};

// ---------------------------------------------------------------------------------------------
// One block per token.  `proj` is the token's row of the fused input projection.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
latent_store_kernel(const T* __restrict__ proj, int ld, int off_kv, int R, int dr, const float* __restrict__ kv_weight,
                    float eps, const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dims,
                    const int* __restrict__ slots, T* __restrict__ pages, int off_q, int q_rank,
                    const float* __restrict__ q_weight, T* __restrict__ q_latent) {
  chain_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * ld;
  if (off_kv >= 0) {
    const T* x = row + off_kv;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
      const float v = Elem<T>::load(x + i);
      ss += v * v;
    }
    const float rs = rsqrtf(block_sum(ss, scratch) / (float)R + eps);
    const int slot = slots[t];
    if (slot >= 0) {
      T* dst = pages + (size_t)slot * (R + dr);
      for (int i = threadIdx.x; i < R; i += blockDim.x) Elem<T>::store(dst + i, Elem<T>::load(x + i) * rs * kv_weight[i]);
      const float pos = (float)positions[t];
      for (int i = threadIdx.x; i < dr / 2; i += blockDim.x) {
        float u = Elem<T>::load(x + R + 2 * i), v = Elem<T>::load(x + R + 2 * i + 1);
        if (2 * i < rot_dims) {
          float sn, cs;
          sincosf(pos * inv_freq[i], &sn, &cs);
          const float a = u * cs - v * sn, b = v * cs + u * sn;
          u = a; v = b;
        }
        Elem<T>::store(dst + R + 2 * i, u);
        Elem<T>::store(dst + R + 2 * i + 1, v);
      }
    }
  }
  if (q_rank > 0) {
    const T* x = row + off_q;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
      const float v = Elem<T>::load(x + i);
      ss += v * v;
    }
    const float rs = rsqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    T* dst = q_latent + (size_t)t * q_rank;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) Elem<T>::store(dst + i, Elem<T>::load(x + i) * rs * q_weight[i]);
  }
}

// q rows [tokens][ld] hold, per head, dn unrotated then dr rotated entries; the rotated ones go, turned,
// to q_lat[token][head][R .. R + dr) as float.
template <typename T>
__global__ void __launch_bounds__(128)
latent_q_rotate_kernel(const T* __restrict__ q, int ld, int H, int dn, int dr, int R, const int* __restrict__ positions,
                       const float* __restrict__ inv_freq, int rot_dims, float* __restrict__ q_lat) {
  chain_wait();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const int half = dr / 2;
  for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    const T* src = q + (size_t)t * ld + (size_t)h * (dn + dr) + dn + 2 * i;
    float u = Elem<T>::load(src), v = Elem<T>::load(src + 1);
    if (2 * i < rot_dims) {
      float sn, cs;
      sincosf(pos * inv_freq[i], &sn, &cs);
      const float a = u * cs - v * sn, b = v * cs + u * sn;
      u = a; v = b;
    }
    float* dst = q_lat + ((size_t)t * H + h) * (R + dr) + R + 2 * i;
    dst[0] = u;
    dst[1] = v;
  }
}

constexpr int kLatWarps = 4;    // (token, head) rows per block: neighbouring heads of a token share its keys in L1
constexpr int kLatKeys = 4;     // keys in flight per warp

// The softmax state of one row after its keys (or one split of them): running maximum, denominator,
// unnormalised sum of latents.  Finishing folds in the sink (a term exp(sink) of the denominator with
// no key and no value) and the head's gate.
__device__ __forceinline__ float finish_factor(float m, float l, const float* sink, int h, float gate_logit, bool gated) {
  float f;
  if (sink) {
    const float s = sink[h], top = fmaxf(m, s);
    const float e = (m == -INFINITY) ? 0.f : expf(m - top);
    f = e / (l * e + expf(s - top));
  } else {
    f = 1.f / l;
  }
  if (gated) f *= 1.f / (1.f + expf(-gate_logit));
  return f;
}

// NI: pairs of the cache row per lane (Dk <= 64 * NI).
template <typename T, int NI>
__global__ void __launch_bounds__(kLatWarps * 32)
latent_attention_kernel(const float* __restrict__ q_lat, const T* __restrict__ pages, const int* __restrict__ block_tables,
                        int max_pages, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                        const T* __restrict__ gate, int gate_ld, const float* __restrict__ sink, T* __restrict__ out,
                        float* __restrict__ part, int first_token, int n_rows, int H, int R, int Dk, int page_size,
                        int split_keys, int n_splits, float scale) {
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kLatWarps + warp;
  if (row >= n_rows) return;                       // warps are independent: no block-wide barrier below
  const int split = blockIdx.y;
  const int t = first_token + row / H, h = row % H;
  const int seq = seq_of_token[t], pos = positions[t];
  const int begin = n_splits > 1 ? split * split_keys : 0;
  const int end = n_splits > 1 ? min(pos + 1, begin + split_keys) : pos + 1;

  float2 q[NI], acc[NI];
  const float* q_row = q_lat + ((size_t)t * H + h) * Dk;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int e = 2 * (lane + 32 * i);
    q[i] = e < Dk ? *reinterpret_cast<const float2*>(q_row + e) : make_float2(0.f, 0.f);
    q[i].x *= scale; q[i].y *= scale;
    acc[i] = make_float2(0.f, 0.f);
  }
  float m = -INFINITY, l = 0.f;
  const int* bt = block_tables + (size_t)seq * max_pages;
  for (int k0 = begin; k0 < end; k0 += kLatKeys) {
    float2 kv[kLatKeys][NI];
    float s[kLatKeys];
#pragma unroll
    for (int j = 0; j < kLatKeys; ++j) {
      const int k = k0 + j < end ? k0 + j : k0;   // (a key past the end is read as the first of the group and masked)
      const T* key = pages + ((size_t)bt[k / page_size] * page_size + k % page_size) * Dk;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const int e = 2 * (lane + 32 * i);
        kv[j][i] = e < Dk ? Pair<T>::load(key + e) : make_float2(0.f, 0.f);
        sum = fmaf(q[i].x, kv[j][i].x, sum);
        sum = fmaf(q[i].y, kv[j][i].y, sum);
      }
      s[j] = sum;
    }
    float top = m;
#pragma unroll
    for (int j = 0; j < kLatKeys; ++j) {
      s[j] = warp_sum(s[j]);
      if (k0 + j >= end) s[j] = -INFINITY;
      top = fmaxf(top, s[j]);
    }
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - top);
    float p[kLatKeys], psum = 0.f;
#pragma unroll
    for (int j = 0; j < kLatKeys; ++j) {
      p[j] = expf(s[j] - top);                    // exp(-inf) = 0 for masked keys
      psum += p[j];
    }
    l = l * alpha + psum;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      float ax = acc[i].x * alpha, ay = acc[i].y * alpha;
#pragma unroll
      for (int j = 0; j < kLatKeys; ++j) {
        ax = fmaf(p[j], kv[j][i].x, ax);
        ay = fmaf(p[j], kv[j][i].y, ay);
      }
      acc[i] = make_float2(ax, ay);
    }
    m = top;
  }
  if (n_splits > 1) {
    float* dst = part + ((size_t)row * n_splits + split) * (R + 2);
    if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int e = 2 * (lane + 32 * i);
      if (e < R) { dst[2 + e] = acc[i].x; dst[3 + e] = acc[i].y; }
    }
    return;
  }
  const float f = finish_factor(m, l, sink, h, gate ? Elem<T>::load(gate + (size_t)t * gate_ld + h) : 0.f, gate != nullptr);
  T* o = out + ((size_t)t * H + h) * R;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int e = 2 * (lane + 32 * i);
    if (e < R) { Elem<T>::store(o + e, acc[i].x * f); Elem<T>::store(o + e + 1, acc[i].y * f); }
  }
}

// One block per row: the splits' states merged in split order (a split the row does not reach has l = 0).
template <typename T>
__global__ void __launch_bounds__(128)
latent_combine_kernel(const float* __restrict__ part, const T* __restrict__ gate, int gate_ld, const float* __restrict__ sink,
                      T* __restrict__ out, int first_token, int H, int R, int n_splits) {
  chain_wait();
  const int row = blockIdx.x;
  const int t = first_token + row / H, h = row % H;
  const float* src = part + (size_t)row * n_splits * (R + 2);
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, src[(size_t)s * (R + 2)]);
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = src[(size_t)s * (R + 2)];
    if (ms != -INFINITY) l += src[(size_t)s * (R + 2) + 1] * expf(ms - m);
  }
  const float f = finish_factor(m, l, sink, h, gate ? Elem<T>::load(gate + (size_t)t * gate_ld + h) : 0.f, gate != nullptr);
  T* o = out + ((size_t)t * H + h) * R;
  for (int e = threadIdx.x; e < R; e += blockDim.x) {
    float sum = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = src[(size_t)s * (R + 2)];
      if (ms != -INFINITY) sum += src[(size_t)s * (R + 2) + 2 + e] * expf(ms - m);
    }
    Elem<T>::store(o + e, sum * f);
  }
}

template <int NI>
void launch_attention(dim3 grid, cudaStream_t stream, const float* q_lat, const elem_t* pages, const int* block_tables,
                      int max_pages, const int* seq_of_token, const int* positions, const elem_t* gate, int gate_ld,
                      const float* sink, elem_t* out, float* part, int first_token, int n_rows, int H, int R, int Dk,
                      int page_size, int split_keys, int n_splits, float scale) {
  launch_chained(latent_attention_kernel<elem_t, NI>, grid, dim3(kLatWarps * 32), 0, stream, q_lat, pages, block_tables,
                 max_pages, seq_of_token, positions, gate, gate_ld, sink, out, part, first_token, n_rows, H, R, Dk, page_size,
                 split_keys, n_splits, scale);
}

}  // namespace

// The token's cache row from its down-projection (when off_kv >= 0) and its query latent (when q_rank > 0).
ERB_EXPORT int erb_latent_store(const void* proj, int n_tokens, int ld, int off_kv, int R, int dr, const float* kv_weight,
                                float eps, const int* positions, const float* inv_freq, int rot_dims, const int* slots,
                                void* pages, int off_q, int q_rank, const float* q_weight, void* q_latent, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (off_kv >= 0 && (R <= 0 || dr < 0 || dr % 2 || rot_dims > dr || rot_dims % 2 || !kv_weight || !slots || !pages ||
                      (rot_dims > 0 && !inv_freq)))
    return fail(ERB_ERR_ARG, "latent_store: bad sizes or missing tensors for the cache row");
  if (q_rank > 0 && (!q_weight || !q_latent)) return fail(ERB_ERR_ARG, "latent_store: the query latent needs a weight and a target");
  launch_chained(latent_store_kernel<elem_t>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (const elem_t*)proj, ld,
                 off_kv, R, dr, kv_weight, eps, positions, inv_freq, rot_dims, slots, (elem_t*)pages, off_q, q_rank, q_weight,
                 (elem_t*)q_latent);
  return check_launch("latent_store");
}

ERB_EXPORT int erb_latent_q_rotate(const void* q, int n_tokens, int ld, int H, int dn, int dr, int R, const int* positions,
                                   const float* inv_freq, int rot_dims, float* q_lat, void* stream) {
  if (n_tokens <= 0 || dr == 0) return ERB_OK;
  if (dr % 2 || rot_dims > dr || rot_dims % 2 || (rot_dims > 0 && !inv_freq))
    return fail(ERB_ERR_ARG, "latent_q_rotate: the rotated part must be even and at least as wide as the rotation");
  launch_chained(latent_q_rotate_kernel<elem_t>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (const elem_t*)q, ld, H, dn,
                 dr, R, positions, inv_freq, rot_dims, q_lat);
  return check_launch("latent_q_rotate");
}

// Rows first_token .. first_token + n_tokens of the batch.  n_splits == 1: every row walks all its keys
// and writes its result; n_splits > 1: keys are cut at multiples of split_keys, `part` (float,
// n_tokens * H * n_splits * (R + 2)) takes the states and a second kernel merges them.
ERB_EXPORT int erb_latent_attention(const float* q_lat, const void* pages, const int* block_tables, int max_pages,
                                    const int* seq_of_token, const int* positions, const void* gate, int gate_ld,
                                    const float* sink, void* out, float* part, int first_token, int n_tokens, int H, int R,
                                    int dr, int page_size, int split_keys, int n_splits, float scale, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  const int Dk = R + dr;
  if (H <= 0 || R <= 0 || R % 2 || dr % 2 || page_size <= 0 || n_splits < 1 || (n_splits > 1 && (!part || split_keys <= 0)))
    return fail(ERB_ERR_ARG, "latent_attention: bad sizes (latent and rotated widths must be even)");
  if (Dk > 640) return fail(ERB_ERR_UNSUPPORTED, "latent_attention: cache rows of %d entries (at most 640)", Dk);
  const int n_rows = n_tokens * H;
  const dim3 grid((n_rows + kLatWarps - 1) / kLatWarps, n_splits);
  cudaStream_t st = (cudaStream_t)stream;
#define ERB_LAT(NI) launch_attention<NI>(grid, st, q_lat, (const elem_t*)pages, block_tables, max_pages, seq_of_token, positions, \
    (const elem_t*)gate, gate_ld, sink, (elem_t*)out, part, first_token, n_rows, H, R, Dk, page_size, split_keys, n_splits, scale)
  if (Dk <= 128) ERB_LAT(2);
  else if (Dk <= 256) ERB_LAT(4);
  else if (Dk <= 384) ERB_LAT(6);
  else ERB_LAT(10);
#undef ERB_LAT
  int rc = check_launch("latent_attention");
  if (rc || n_splits == 1) return rc;
  launch_chained(latent_combine_kernel<elem_t>, dim3(n_rows), dim3(128), 0, st, (const float*)part, (const elem_t*)gate, gate_ld,
                 sink, (elem_t*)out, first_token, H, R, n_splits);
  return check_launch("latent_combine");
}
