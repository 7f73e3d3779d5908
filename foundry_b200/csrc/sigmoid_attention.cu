// Grouped-query attention whose weights are sigmoids, not a softmax, over the
// keys of the query's own chunk of the sequence; and the kernel in front of it.
//
//   q, k: per head  x / sqrt(mean(x^2) + eps) * w   (w [dim], the same for every head;
//         absent: no weight), then rotated on the first `rot` elements of a head:
//         (x_i, x_{i + rot/2}) at position p turn by the angle p * f_i
//   v:    per head  x / sqrt(mean(x^2) + eps)  where `value_norm`; cached so
//   s_ij = (q_i . k_j) * scale + bias[head]
//   j visible to i  iff  j <= i and floor(i / chunk) == floor(j / chunk)   (chunk 0: j <= i)
//   o_i = out_scale * gate_i[head] * sum_j sigmoid(s_ij) v_j ,  gate = sigmoid(raw gate)  (absent: 1)
//
// The weights are not normalised over the keys, so there is no running maximum
// and no sum to divide by: a key's share does not depend on the other keys.
// Every constant is a parameter. Positions are the tokens' own, and a chunk's
// borders are multiples of `chunk` in them, whatever the step brings. Angles are
// the double-precision product of the position and a double-precision frequency.
//
// This file holds the CUDA-core forms (32-bit arithmetic, any sizes): a block
// per (token, query head) whose warps take the visible keys 32 at a time, a
// lane a key for the scores and a lane a value element for the sums, the
// warps' shares added in warp order.
#include "common.cuh"

namespace {
constexpr int SG_WARPS = 4;

template <typename T>
__device__ __forceinline__ void sg_load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void sg_load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldcg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcg(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void sg_load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// One block a token. Rows of `qkv` are [q: H x dim | k: G x dim | v: G x vdim] in
// float32. Queries go to `q_out` in the activation type, keys and values into the
// token's cache row. `qk_norm` 0 leaves queries and keys as they are; `interleaved`
// 1 turns elements (2i, 2i + 1) instead of (i, i + rot / 2); G may be 0 (a mixer that
// reads another's keys and values has queries only).
template <typename T>
__global__ void head_norm_rope_cache_kernel(const float* qkv, long long ld, T* __restrict__ q_out,
                                            const float* __restrict__ wq,
                                            const float* __restrict__ wk, float eps,
                                            int qk_norm, int value_norm,
                                            const double* __restrict__ freq, int rot,
                                            int interleaved, const int* __restrict__ positions,
                                            const int* __restrict__ seq_of_token,
                                            const int* __restrict__ page_table, int max_pages,
                                            T* __restrict__ k_cache, T* __restrict__ v_cache,
                                            long long k_page, long long k_head, long long v_page,
                                            long long v_head, int H, int G, int dim, int vdim,
                                            int write_cache, int head_floats) {
  fb_pdl_launch();
  fb_pdl_wait();
  extern __shared__ float sg_smem[];  // cos [rot/2] | sin [rot/2] | a head's elements per warp
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const int pos = seq >= 0 ? positions[t] : 0;
  const int half = rot / 2;
  float* cs = sg_smem;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const double angle = (double)pos * freq[i];
    cs[i] = (float)cos(angle);
    cs[half + i] = (float)sin(angle);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float* buf = sg_smem + rot + (size_t)warp * head_floats;
  const float* row = qkv + (size_t)t * ld;
  long long page = 0;
  int r_in_page = 0;
  const bool cached = write_cache && seq >= 0;
  if (cached) {
    page = page_table[(size_t)seq * max_pages + pos / FB_PAGE];
    r_in_page = pos % FB_PAGE;
  }
  // a warp a head; a token's heads (queries, keys, values) are spread over blockIdx.y
  for (int u = blockIdx.y * nwarps + warp; u < H + 2 * G; u += gridDim.y * nwarps) {
    const bool is_q = u < H, is_k = !is_q && u < H + G;
    const int g = is_q ? u : (is_k ? u - H : u - H - G);
    const int n = (is_q || is_k) ? dim : vdim;
    const float* src = is_q ? row + (size_t)g * dim
                            : is_k ? row + (size_t)H * dim + (size_t)g * dim
                                   : row + (size_t)(H + G) * dim + (size_t)g * vdim;
    float ss = 0.f;
    for (int d = lane; d < n; d += 32) {
      const float x = __ldcg(src + d);
      buf[d] = x;
      ss = fmaf(x, x, ss);
    }
    ss = fb_warp_sum(ss);
    const bool normed = (is_q || is_k) ? qk_norm != 0 : value_norm != 0;
    const float r = normed ? 1.0f / sqrtf(ss / (float)n + eps) : 1.0f;
    const float* w = is_q ? wq : is_k ? wk : nullptr;
    __syncwarp();
    for (int d = lane; d < n; d += 32) buf[d] = buf[d] * r * (w != nullptr ? w[d] : 1.0f);
    __syncwarp();
    if (is_q || is_k) {
      for (int i = lane; i < half; i += 32) {
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
        const float a = buf[ia], b = buf[ib];
        const float c = cs[i], s = cs[half + i];
        buf[ia] = a * c - b * s;
        buf[ib] = b * c + a * s;
      }
      __syncwarp();
    }
    if (is_q) {
      T* dst = q_out + ((size_t)t * H + g) * dim;
      for (int d = lane; d < n; d += 32) dst[d] = fb_from_float<T>(buf[d]);
    } else if (cached) {
      T* dst = is_k ? k_cache + page * k_page + (long long)g * k_head + (long long)r_in_page * dim
                    : v_cache + page * v_page + (long long)g * v_head + (long long)r_in_page * vdim;
      for (int d = lane; d < n; d += 32) dst[d] = fb_from_float<T>(buf[d]);
    }
    __syncwarp();
  }
}

template <typename T>
__global__ void __launch_bounds__(SG_WARPS * 32)
attention_sigmoid_kernel(const T* q, long long q_stride, T* __restrict__ out, long long out_stride,
                         const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                         const int* __restrict__ page_table, int max_pages, const T* k_cache,
                         const T* v_cache, long long k_page, long long k_head, long long v_page,
                         long long v_head, const float* __restrict__ head_bias, const float* gate,
                         long long gate_ld, float scale, float out_scale, int chunk, int H, int G,
                         int D, int VD, int kvec) {
  fb_pdl_wait();
  extern __shared__ float sg_att[];  // q [D] | the warps' shares [SG_WARPS][VD]
  constexpr int NACC = 8;            // value elements a lane sums (values of up to 256)
  float* qs = sg_att;
  float* shares = sg_att + D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, a = blockIdx.y;
  const int seq = seq_of_token[t];
  T* o = out + (size_t)t * out_stride + (size_t)a * VD;
  if (seq < 0) {  // padding token: defined output, no cache access
    for (int d = threadIdx.x; d < VD; d += blockDim.x) o[d] = fb_from_float<T>(0.f);
    return;
  }
  const int pos = positions[t];
  const int g = a / (H / G);
  const T* qrow = q + (size_t)t * q_stride + (size_t)a * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = fb_load_coherent<T>(qrow + d);
  __syncthreads();
  const int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
  const float bias = head_bias != nullptr ? head_bias[a] : 0.f;
  const int* pages = page_table + (size_t)seq * max_pages;
  const T* kbase = k_cache + (long long)g * k_head;
  const T* vbase = v_cache + (long long)g * v_head;
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  for (int j0 = lo + warp * 32; j0 <= pos; j0 += SG_WARPS * 32) {
    const int j = j0 + lane;
    float w = 0.f;
    long long v_off = 0;
    if (j <= pos) {
      const long long page = pages[j / FB_PAGE];
      const int r = j % FB_PAGE;
      v_off = page * v_page + (long long)r * VD;
      const T* krow = kbase + page * k_page + (long long)r * D;
      float dot = 0.f;
      if (kvec) {
        for (int d = 0; d < D; d += 8) {
          float kv[8];
          sg_load8<T>(krow + d, kv);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(qs[d + e], kv[e], dot);
        }
      } else {
        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], fb_load_coherent<T>(krow + d), dot);
      }
      w = 1.0f / (1.0f + expf(-(dot * scale + bias)));
    }
    const int n = min(32, pos + 1 - j0);
    for (int jj = 0; jj < n; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, w, jj);
      const long long off = __shfl_sync(0xffffffffu, v_off, jj);
      const T* vrow = vbase + off;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < VD) acc[i] = fmaf(pj, fb_load_coherent<T>(vrow + d), acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < VD) shares[warp * VD + d] = acc[i];
  }
  __syncthreads();
  float gz = out_scale;
  if (gate != nullptr) gz *= 1.0f / (1.0f + expf(-__ldcg(gate + (size_t)t * gate_ld + a)));
  for (int d = threadIdx.x; d < VD; d += blockDim.x) {
    float s = shares[d];
#pragma unroll
    for (int wi = 1; wi < SG_WARPS; ++wi) s += shares[wi * VD + d];
    o[d] = fb_from_float<T>(s * gz);
  }
}

// ---------------------------------------------- few tokens, each with many keys
// A block per (token, key head, run of keys): the query heads that share the key
// head (up to RMAX at a time) ride on one walk over the run, so a key row and a
// value row are loaded once for all of them. A warp takes 32 keys at a time, a lane
// a key for the scores; for the sums a lane holds NACC value elements of each head
// and the value rows of four keys are in flight at once. The warps' shares are
// added in warp order, the runs' shares (`partial` [runs, T, H, VD], when there is
// more than one run) in run order by the kernel below: no result depends on timing.
constexpr int SG_RMAX = 4;

// A 16-byte piece of a row as floats.
template <typename T>
__device__ __forceinline__ void sg_load_piece(const T* p, float (&v)[16 / sizeof(T)]);
template <>
__device__ __forceinline__ void sg_load_piece<float>(const float* p, float (&v)[4]) {
  const float4 a = __ldcg(reinterpret_cast<const float4*>(p));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <>
__device__ __forceinline__ void sg_load_piece<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  sg_load8<__nv_bfloat16>(p, v);
}

// VEC: value rows are read in 16-byte pieces, `ppr` lanes a row (a power of two), so that a
// warp's load instruction fetches 32 / ppr rows and eight of them are in flight; a lane then
// holds one piece's columns for every (32 / ppr)-th key, and the lanes of a column add up at
// the end. Otherwise a lane holds NACC single columns of every key.
template <typename T, int NACC, bool VEC>
__global__ void __launch_bounds__(512)
attention_sigmoid_group_kernel(const T* q, long long q_stride, T* __restrict__ out,
                               long long out_stride, float* __restrict__ partial,
                               const int* __restrict__ positions,
                               const int* __restrict__ seq_of_token,
                               const int* __restrict__ page_table, int max_pages, const T* k_cache,
                               const T* v_cache, long long k_page, long long k_head,
                               long long v_page, long long v_head,
                               const float* __restrict__ head_bias, const float* gate,
                               long long gate_ld, float scale, float out_scale, int chunk, int H,
                               int G, int D, int VD, int kvec, int span, int n_tokens, int ppr) {
  fb_pdl_wait();
  constexpr int EPV = 16 / sizeof(T);  // elements a piece holds
  extern __shared__ float sg_grp[];  // q [SG_RMAX][D] | the warps' shares [warps][SG_RMAX][VD]
  float* qs = sg_grp;
  float* shares = sg_grp + SG_RMAX * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int t = blockIdx.x, rep = H / G;
  const int parts = (rep + SG_RMAX - 1) / SG_RMAX;
  const int g = blockIdx.y / parts;
  const int a0 = g * rep + (blockIdx.y % parts) * SG_RMAX;     // first query head of the block
  const int na = min(SG_RMAX, g * rep + rep - a0);             // how many it has
  const int runs = gridDim.z, z = blockIdx.z;
  const int seq = seq_of_token[t];
  int lo = 0, hi = -1;  // this block's keys, both ends included
  if (seq >= 0) {
    const int pos = positions[t];
    const int first = chunk > 0 ? (pos / chunk) * chunk : 0;
    lo = first + z * span;
    hi = min(pos, lo + span - 1);
  }
  for (int i = threadIdx.x; i < SG_RMAX * D; i += blockDim.x) {
    const int r = i / D, d = i - r * D;
    qs[i] = (r < na && hi >= lo)
                ? fb_load_coherent<T>(q + (size_t)t * q_stride + (size_t)(a0 + r) * D + d) : 0.f;
  }
  __syncthreads();
  float bias[SG_RMAX];
#pragma unroll
  for (int r = 0; r < SG_RMAX; ++r) bias[r] = (head_bias != nullptr && r < na) ? head_bias[a0 + r] : 0.f;
  const int* pages = page_table + (size_t)(seq < 0 ? 0 : seq) * max_pages;
  const T* kbase = k_cache + (long long)g * k_head;
  const T* vbase = v_cache + (long long)g * v_head;
  constexpr int NA = VEC ? EPV : NACC;
  float acc[SG_RMAX][NA];
#pragma unroll
  for (int r = 0; r < SG_RMAX; ++r)
#pragma unroll
    for (int i = 0; i < NA; ++i) acc[r][i] = 0.f;
  const int piece = VEC ? lane % ppr : 0, sub = VEC ? lane / ppr : 0, rows_at_once = VEC ? 32 / ppr : 1;
  for (int j0 = lo + warp * 32; j0 <= hi; j0 += nwarps * 32) {
    const int j = j0 + lane;
    float w[SG_RMAX];
#pragma unroll
    for (int r = 0; r < SG_RMAX; ++r) w[r] = 0.f;
    long long v_off = 0;
    if (j <= hi) {
      const long long page = pages[j / FB_PAGE];
      const int row = j % FB_PAGE;
      v_off = page * v_page + (long long)row * VD;
      const T* krow = kbase + page * k_page + (long long)row * D;
      float dot[SG_RMAX];
#pragma unroll
      for (int r = 0; r < SG_RMAX; ++r) dot[r] = 0.f;
      if (kvec) {
#pragma unroll 4
        for (int d = 0; d < D; d += 8) {
          float kv[8];
          sg_load8<T>(krow + d, kv);
#pragma unroll
          for (int r = 0; r < SG_RMAX; ++r)
#pragma unroll
            for (int e = 0; e < 8; ++e) dot[r] = fmaf(qs[r * D + d + e], kv[e], dot[r]);
        }
      } else {
        for (int d = 0; d < D; ++d) {
          const float kd = fb_load_coherent<T>(krow + d);
#pragma unroll
          for (int r = 0; r < SG_RMAX; ++r) dot[r] = fmaf(qs[r * D + d], kd, dot[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < SG_RMAX; ++r) w[r] = 1.0f / (1.0f + expf(-(dot[r] * scale + bias[r])));
    }
    const int n = min(32, hi + 1 - j0);
    if constexpr (VEC) {
      for (int jj = 0; jj < n; jj += 8 * rows_at_once) {
        float vals[8][EPV];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int row = jj + u * rows_at_once + sub;  // which of the 32 keys
          const long long off = __shfl_sync(0xffffffffu, v_off, row & 31);
          if (row < n) {  // a row past the run is not read: it may hold anything
            sg_load_piece<T>(vbase + off + piece * EPV, vals[u]);
          } else {
#pragma unroll
            for (int e = 0; e < EPV; ++e) vals[u][e] = 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int row = jj + u * rows_at_once + sub;
#pragma unroll
          for (int r = 0; r < SG_RMAX; ++r) {
            const float pj = __shfl_sync(0xffffffffu, w[r], row & 31);
            const float pw = row < n ? pj : 0.f;
#pragma unroll
            for (int e = 0; e < EPV; ++e) acc[r][e] = fmaf(pw, vals[u][e], acc[r][e]);
          }
        }
      }
    } else
    for (int jj = 0; jj < n; jj += 4) {
      float vals[4][NACC];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long off = __shfl_sync(0xffffffffu, v_off, (jj + u) & 31);
        const bool there = jj + u < n;  // a row past the run is not read: it may hold anything
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
          const int d = lane + 32 * i;
          vals[u][i] = (there && d < VD) ? fb_load_coherent<T>(vbase + off + d) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int r = 0; r < SG_RMAX; ++r) {
          const float pj = __shfl_sync(0xffffffffu, w[r], (jj + u) & 31);
          const float pw = jj + u < n ? pj : 0.f;
#pragma unroll
          for (int i = 0; i < NACC; ++i) acc[r][i] = fmaf(pw, vals[u][i], acc[r][i]);
        }
      }
    }
  }
  if constexpr (VEC) {
#pragma unroll
    for (int r = 0; r < SG_RMAX; ++r)
#pragma unroll
      for (int e = 0; e < EPV; ++e) {
        float v = acc[r][e];
        for (int o = ppr; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane < ppr) shares[((size_t)warp * SG_RMAX + r) * VD + piece * EPV + e] = v;
      }
  } else {
#pragma unroll
    for (int r = 0; r < SG_RMAX; ++r)
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < VD) shares[((size_t)warp * SG_RMAX + r) * VD + d] = acc[r][i];
      }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < na * VD; i += blockDim.x) {
    const int r = i / VD, d = i - r * VD;
    float s = shares[(size_t)r * VD + d];
    for (int wi = 1; wi < nwarps; ++wi) s += shares[((size_t)wi * SG_RMAX + r) * VD + d];
    const int a = a0 + r;
    if (runs > 1) {
      partial[(((size_t)z * n_tokens + t) * H + a) * VD + d] = s;
    } else {
      float gz = out_scale;
      if (gate != nullptr) gz *= 1.0f / (1.0f + expf(-__ldcg(gate + (size_t)t * gate_ld + a)));
      // (a padding token: a defined output whatever its gate row holds)
      out[(size_t)t * out_stride + (size_t)a * VD + d] = fb_from_float<T>(seq < 0 ? 0.f : s * gz);
    }
  }
}

// out[t, head] = out_scale * sigmoid(gate[t, head]) * the sum over the runs, in run order
template <typename T>
__global__ void attention_sigmoid_runs_kernel(const float* partial, int runs, T* __restrict__ out,
                                              long long out_stride, const float* gate,
                                              long long gate_ld, float out_scale, int n_tokens,
                                              int H, int VD) {
  fb_pdl_wait();
  const int t = blockIdx.x, a = blockIdx.y;
  float gz = out_scale;
  if (gate != nullptr) gz *= 1.0f / (1.0f + expf(-__ldcg(gate + (size_t)t * gate_ld + a)));
  for (int d = threadIdx.x; d < VD; d += blockDim.x) {
    float s = 0.f;
    for (int z = 0; z < runs; ++z) s += __ldcg(partial + (((size_t)z * n_tokens + t) * H + a) * VD + d);
    out[(size_t)t * out_stride + (size_t)a * VD + d] = fb_from_float<T>(s * gz);
  }
}
}  // namespace

FB_API int fb_head_norm_rope_cache_write(const float* qkv, long long ld, void* q_out, int dtype,
                                         const float* wq, const float* wk, float eps,
                                         int qk_norm, int value_norm, const double* freq,
                                         int rot, int interleaved, const int* positions,
                                         const int* seq_of_token,
                                         const int* page_table, int max_pages, void* k_cache,
                                         void* v_cache, long long k_page, long long k_head,
                                         long long v_page, long long v_head, int T, int H, int G,
                                         int dim, int vdim, int write_cache, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && G >= 0 && dim > 0 && vdim > 0, "head_norm_rope_cache_write: bad sizes");
  FB_REQUIRE(G > 0 || !write_cache, "head_norm_rope_cache_write: no keys to write");
  FB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dim && (rot == 0 || freq != nullptr),
             "head_norm_rope_cache_write: %d rotated elements of %d", rot, dim);
  FB_REQUIRE(ld >= (long long)(H + G) * dim + (long long)G * vdim,
             "head_norm_rope_cache_write: rows of %lld are too short", ld);
  if (T == 0) return 0;
  const int heads = H + 2 * G;
  const int warps = heads < 8 ? heads : 8;
  const int head_floats = dim > vdim ? dim : vdim;
  const size_t smem = (size_t)(rot + warps * head_floats) * 4;
  FB_REQUIRE(smem <= 48 * 1024, "head_norm_rope_cache_write: heads of %d do not fit", head_floats);
  const int parts = T <= 256 ? (heads + warps - 1) / warps : 1;  // few tokens: more blocks
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(head_norm_rope_cache_kernel<E>, dim3(T, parts), dim3(warps * 32),
      smem, stream, qkv, ld, (E*)q_out, wq, wk, eps, qk_norm, value_norm, freq, rot, interleaved,
      positions,
      seq_of_token, page_table, max_pages, (E*)k_cache, (E*)v_cache, k_page, k_head, v_page,
      v_head, H, G, dim, vdim, write_cache, head_floats)));
  return fb_check_launch("head_norm_rope_cache_write");
}

FB_API int fb_attention_sigmoid(const void* q, long long q_stride, void* out, long long out_stride,
                                int dtype, const int* positions, const int* seq_of_token,
                                const int* page_table, int max_pages, const void* k_cache,
                                const void* v_cache, long long k_page, long long k_head,
                                long long v_page, long long v_head, const float* head_bias,
                                const float* gate, long long gate_ld, float scale,
                                float out_scale, int chunk, int T, int H, int G, int dim, int vdim, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && chunk >= 0,
             "attention_sigmoid: bad sizes");
  FB_REQUIRE(vdim <= 256, "attention_sigmoid: values of %d exceed 256", vdim);
  FB_REQUIRE(H <= 65535, "attention_sigmoid: %d heads", H);
  if (T == 0) return 0;
  const size_t smem = (size_t)(dim + SG_WARPS * vdim) * 4;
  FB_REQUIRE(smem <= 48 * 1024, "attention_sigmoid: heads of %d do not fit", dim);
  const size_t esize = dtype == FB_BF16 ? 2 : 4;
  const int kvec = (dim * esize) % 16 == 0 && ((uintptr_t)k_cache % 16) == 0 &&
                   ((size_t)k_page * esize) % 16 == 0 && ((size_t)k_head * esize) % 16 == 0 &&
                   dim % 8 == 0;
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_sigmoid_kernel<E>, dim3(T, H),
      dim3(SG_WARPS * 32), smem, stream, (const E*)q, q_stride, (E*)out, out_stride, positions,
      seq_of_token, page_table, max_pages, (const E*)k_cache, (const E*)v_cache, k_page, k_head,
      v_page, v_head, head_bias, gate, gate_ld, scale, out_scale, chunk, H, G, dim, vdim, kvec)));
  return fb_check_launch("attention_sigmoid");
}

// The form for steps of few tokens (one a sequence, say): see the kernel. `span`: keys a
// run holds; `runs`: how many runs the longest visible range of the step is cut into
// (the caller's bound); `partial`: float32 [runs, T, H, vdim] when runs > 1.
FB_API int fb_attention_sigmoid_group(const void* q, long long q_stride, void* out,
                                      long long out_stride, int dtype, float* partial,
                                      const int* positions, const int* seq_of_token,
                                      const int* page_table, int max_pages, const void* k_cache,
                                      const void* v_cache, long long k_page, long long k_head,
                                      long long v_page, long long v_head, const float* head_bias,
                                      const float* gate, long long gate_ld, float scale,
                                      float out_scale, int chunk, int span, int runs, int T, int H,
                                      int G, int dim, int vdim, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && chunk >= 0,
             "attention_sigmoid_group: bad sizes");
  FB_REQUIRE(vdim <= 256, "attention_sigmoid_group: values of %d exceed 256", vdim);
  FB_REQUIRE(span > 0 && runs >= 1 && runs <= 65535 && (runs == 1 || partial != nullptr),
             "attention_sigmoid_group: %d runs of %d keys", runs, span);
  if (T == 0) return 0;
  const int parts = (H / G + SG_RMAX - 1) / SG_RMAX;
  FB_REQUIRE((long long)G * parts <= 65535, "attention_sigmoid_group: %d key heads", G);
  int warps = 16;  // as many as the shares leave room for
  while (warps > 1 && (size_t)(SG_RMAX * dim + warps * SG_RMAX * vdim) * 4 > 48 * 1024) warps /= 2;
  const size_t smem = (size_t)(SG_RMAX * dim + warps * SG_RMAX * vdim) * 4;
  FB_REQUIRE(smem <= 48 * 1024, "attention_sigmoid_group: heads of %d do not fit", dim);
  const size_t esize = dtype == FB_BF16 ? 2 : 4;
  const int kvec = (dim * esize) % 16 == 0 && ((uintptr_t)k_cache % 16) == 0 &&
                   ((size_t)k_page * esize) % 16 == 0 && ((size_t)k_head * esize) % 16 == 0 &&
                   dim % 8 == 0;
  const dim3 grid(T, G * parts, runs), block(warps * 32);
  // value rows in 16-byte pieces: a power of two of them a row, at most one a lane
  const size_t row_bytes = (size_t)vdim * esize;
  int ppr = 0;
  if (row_bytes % 16 == 0 && row_bytes / 16 <= 32 && ((row_bytes / 16) & (row_bytes / 16 - 1)) == 0 &&
      ((uintptr_t)v_cache % 16) == 0 && ((size_t)v_page * esize) % 16 == 0 &&
      ((size_t)v_head * esize) % 16 == 0)
    ppr = (int)(row_bytes / 16);
#define FB_SG_GROUP(E, NACC, VEC)                                                                  \
  fb_launch(attention_sigmoid_group_kernel<E, NACC, VEC>, grid, block, smem, stream, (const E*)q,  \
            q_stride, (E*)out, out_stride, partial, positions, seq_of_token, page_table, max_pages, \
            (const E*)k_cache, (const E*)v_cache, k_page, k_head, v_page, v_head, head_bias, gate, \
            gate_ld, scale, out_scale, chunk, H, G, dim, vdim, kvec, span, T, ppr)
  FB_DISPATCH_DTYPE(dtype, E, {
    if (ppr > 0) FB_SG_GROUP(E, 1, true);
    else if (vdim <= 32) FB_SG_GROUP(E, 1, false);
    else if (vdim <= 64) FB_SG_GROUP(E, 2, false);
    else if (vdim <= 128) FB_SG_GROUP(E, 4, false);
    else FB_SG_GROUP(E, 8, false);
  });
#undef FB_SG_GROUP
  int rc = fb_check_launch("attention_sigmoid_group");
  if (rc != 0 || runs == 1) return rc;
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_sigmoid_runs_kernel<E>, dim3(T, H), dim3(64), 0,
      stream, (const float*)partial, runs, (E*)out, out_stride, gate, gate_ld, out_scale, T, H,
      vdim)));
  return fb_check_launch("attention_sigmoid_runs");
}
