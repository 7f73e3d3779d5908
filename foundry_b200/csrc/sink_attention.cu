// Grouped-query attention over the paged cache with a distance bias, a sliding
// window that keeps the first tokens, and a softmax with a sink; with a norm
// of the whole query and key projections in front of it.
//
//   q' = q / sqrt(mean(q^2) + eps) * wq     over ALL query rows of a token at once
//   k' = k / sqrt(mean(k^2) + eps) * wk     (before the split into heads)
//   s_ij = (q'_i . k'_j) * scale - slope_h * (i - j),  slope_h = 2^(-steep (h+1) / H)
//   j visible to i  iff  j <= i and (i - j < window or j < keep_first)
//   p_ij = exp(s_ij) / (sink + sum_j exp(s_ij)),  sink = 1 or 0: one more term exp(0)
//          in the sum, which adds nothing to the output
//   o_i = sum_j p_ij v_j
//
// Every constant is a parameter: window 0 = all earlier keys, steep 0 = no bias,
// sink 0 = the plain softmax. Keys have `dim` elements and values `vdim`; the
// two caches have strides of their own. Positions are the tokens' own, so the
// bias of a kept token is by the distance it really has.
//
// More rules of the same kernels, each off unless asked for (see `ScoreRule`): a cap
// on the scores, softcap * tanh(s / softcap); a sink whose score is a learned number
// per head instead of 0; two maps a head (two query vectors against two key vectors
// side by side in a key row, two softmaxes over the same values, joined as
// (a1 - lambda a2) / rms * scale in the kernel's epilogue); values that are the first
// elements of the key rows (a cache of latent rows). Beside them the small kernels in
// front of such attentions: queries times a temperature that grows with the position
// plus the cache write; the norms and the rotation of a latent projection plus its
// cache row; the split of query heads into a plain and a rotated part.
//
// This file holds the CUDA-core forms (32-bit arithmetic, any sizes): one warp
// per (token, query head) walking the kept prefix and then the window, either
// straight from the cache or, for rows of whole 16-byte pieces, from a chunk's rows
// staged in shared memory once for the heads that share a key head.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_QD = 1024;  // elements of a query head over all its maps

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldcg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcg(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// ------------------------------------------------ whole-projection norm + cache
template <typename T>
__global__ void qk_norm_cache_kernel(const float* qkv, long long ld, T* __restrict__ q_out,
                                     const float* __restrict__ wq, const float* __restrict__ wk,
                                     float eps, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token,
                                     const int* __restrict__ page_table, int max_pages,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     long long k_page, long long k_head, long long v_page,
                                     long long v_head, int H, int G, int dim, int vdim,
                                     int write_cache) {
  fb_pdl_launch();
  fb_pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const int nq = H * dim, nk = G * dim, nv = G * vdim;
  const float* row = qkv + (size_t)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) {
    const float v = __ldcg(row + i);
    sq += v * v;
  }
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const float v = __ldcg(row + nq + i);
    sk += v * v;
  }
  sq = fb_block_sum(sq, scratch);
  sk = fb_block_sum(sk, scratch);
  const float rq = 1.0f / sqrtf(sq / (float)nq + eps);
  const float rk = 1.0f / sqrtf(sk / (float)nk + eps);
  T* qo = q_out + (size_t)t * nq;
  for (int i = threadIdx.x; i < nq; i += blockDim.x)
    qo[i] = fb_from_float<T>(__ldcg(row + i) * rq * wq[i]);
  if (!write_cache || seq < 0) return;
  const int pos = positions[t];
  const long long page = page_table[(size_t)seq * max_pages + pos / FB_PAGE];
  const int r = pos % FB_PAGE;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int g = i / dim, d = i - g * dim;
    k_cache[page * k_page + g * k_head + (long long)r * dim + d] =
        fb_from_float<T>(__ldcg(row + nq + i) * rk * wk[i]);
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const int g = i / vdim, d = i - g * vdim;
    v_cache[page * v_page + g * v_head + (long long)r * vdim + d] =
        fb_from_float<T>(__ldcg(row + nq + nk + i));
  }
}

// ---------------------------------------------------------------- attention
// How a score is made and what joins the softmax's sum, all as parameters:
//   s = cap(q . k * scale) - slope_h * (i - j),   cap(x) = softcap * tanh(x / softcap) (softcap 0: x)
//   sink 0: none; 1: one more term exp(0); 2: one more term exp(sink_logit[head])
// With two maps (MAPS = 2) a query head has two query vectors and a key row two key
// vectors side by side, [map 1 | map 2]; each map is an attention of its own over the
// same value rows, and the head's output is
//   o = a1 - lambda * a2;   o <- o / sqrt(mean(o^2) + post_eps) * post_scale.
struct ScoreRule {
  int window, keep_first, sink;
  const float* sink_logit;
  float scale, steep, softcap;
  float lambda, post_eps, post_scale;
};

__device__ __forceinline__ float capped(float s, float cap) {
  return cap > 0.f ? cap * tanhf(s / cap) : s;
}

// Value rows lie `v_row` elements apart and key rows `k_row` (so values may be a
// part of the key rows: a cache of latent rows read as keys and as values).
// VEC (value size a multiple of 8, 16-byte aligned value rows): a value row is
// read as 16-byte pieces by `lpr` neighbouring lanes and 32 / lpr keys are worked at
// a time, every lane's loads of a chunk independent of one another; the lanes that
// share a piece add their sums up once, at the end. Rows of more than 256 values
// take several pieces a lane (NACC / 8). Otherwise a lane owns the elements lane,
// lane + 32, ... and keys go one by one. NACC: value elements a lane accumulates.
template <typename T, bool VEC, int MAPS, int NACC>
__global__ void __launch_bounds__(WARPS * 32)
attention_sink_kernel(const T* q, long long q_stride, T* __restrict__ out, long long out_stride,
                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                      const int* __restrict__ page_table, int max_pages, const T* k_cache,
                      const T* v_cache, long long k_page, long long k_head, long long v_page,
                      long long v_head, int k_row, int v_row, ScoreRule rule, int H, int G, int D,
                      int VD, int splits, float* __restrict__ partial, int lpr, int kvec) {
  fb_pdl_wait();
  extern __shared__ float qs_all[];  // [WARPS][MAPS * D]
  constexpr int PIECES = NACC / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = qs_all + (size_t)warp * MAPS * D;
  const int t = blockIdx.x;
  const int a = blockIdx.y * WARPS + warp;
  if (a >= H) return;
  const int seq = seq_of_token[t];
  T* o = out + (size_t)t * out_stride + (size_t)a * VD;
  if (seq < 0) {  // padding token: defined output, no cache access
    for (int d = lane; d < VD; d += 32) o[d] = fb_from_float<T>(0.f);
    return;
  }
  const int pos = positions[t];
  const int g = a / (H / G);
  const T* qrow = q + (size_t)t * q_stride + (size_t)a * MAPS * D;
  for (int d = lane; d < MAPS * D; d += 32) qs[d] = fb_load_coherent<T>(qrow + d);
  __syncwarp();
  const float slope = rule.steep > 0.f ? exp2f(-rule.steep * (float)(a + 1) / (float)H) : 0.f;
  const int lo = (rule.window > 0 && pos - rule.window + 1 > 0) ? pos - rule.window + 1 : 0;
  const int kept = min(rule.keep_first, lo);  // keys [0, kept) lie in front of the window
  const int* pages = page_table + (size_t)seq * max_pages;
  const T* kbase = k_cache + (long long)g * k_head;
  const T* vbase = v_cache + (long long)g * v_head;

  // With `splits` > 1 the visible keys (the kept ones, then the window's) are cut into
  // that many runs; block z takes run z and leaves (max, sum, weighted values) per map
  // for `attention_sink_merge_kernel`, which also adds the sink and combines the maps.
  const int total = kept + (pos + 1 - lo);
  const int i0 = (int)((long long)total * blockIdx.z / splits);
  const int i1 = (int)((long long)total * (blockIdx.z + 1) / splits);
  // the sink is one more term of the sum: the running maximum starts at its score, the sum at 1
  const bool own_sink = rule.sink && splits == 1;
  const float sink_score = rule.sink == 2 ? rule.sink_logit[a] : 0.f;
  float m[MAPS], l[MAPS];
  float acc[MAPS][NACC];
#pragma unroll
  for (int mm = 0; mm < MAPS; ++mm) {
    m[mm] = own_sink ? sink_score : -INFINITY;
    l[mm] = own_sink ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[mm][i] = 0.f;
  }

  for (int range = 0; range < 2; ++range) {
    const int begin = range == 0 ? min(i0, kept) : lo + max(i0 - kept, 0);
    const int end = range == 0 ? min(i1, kept) : lo + max(i1 - kept, 0);  // exclusive
    for (int j0 = begin; j0 < end; j0 += 32) {
      const int j = j0 + lane;
      float s[MAPS];
#pragma unroll
      for (int mm = 0; mm < MAPS; ++mm) s[mm] = -INFINITY;
      long long v_off = 0;
      if (j < end) {
        const long long page = pages[j / FB_PAGE];
        const int r = j % FB_PAGE;
        v_off = page * v_page + (long long)r * v_row;
        const T* krow = kbase + page * k_page + (long long)r * k_row;
#pragma unroll
        for (int mm = 0; mm < MAPS; ++mm) {
          const float* qm = qs + mm * D;
          const T* km = krow + mm * D;
          float dot = 0.f;
          if (kvec) {  // key rows of whole 16-byte pieces, four loads in flight at a time
            for (int d = 0; d < D; d += 32) {
              float kv[4][8];
#pragma unroll
              for (int u = 0; u < 4; ++u)
                if (d + u * 8 < D) load8<T>(km + d + u * 8, kv[u]);
#pragma unroll
              for (int u = 0; u < 4; ++u)
                if (d + u * 8 < D)
#pragma unroll
                  for (int e = 0; e < 8; ++e) dot = fmaf(qm[d + u * 8 + e], kv[u][e], dot);
            }
          } else {
            for (int d = 0; d < D; ++d) dot = fmaf(qm[d], fb_load_coherent<T>(km + d), dot);
          }
          s[mm] = capped(dot * rule.scale, rule.softcap) - slope * (float)(pos - j);
        }
      }
      float p[MAPS];
#pragma unroll
      for (int mm = 0; mm < MAPS; ++mm) {
        const float m_new = fmaxf(m[mm], fb_warp_max(s[mm]));
        const float corr = expf(m[mm] - m_new);  // exp(-inf) = 0 on a first chunk without sink
        p[mm] = (j < end) ? expf(s[mm] - m_new) : 0.f;
        l[mm] = l[mm] * corr + fb_warp_sum(p[mm]);
        m[mm] = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[mm][i] *= corr;
      }
      const int n = min(32, end - j0);
      if (VEC) {
        const int sub = lane / lpr, ks = 32 / lpr;
        // U groups of keys at a time, the loads of all of them issued before the first sum:
        // a lane's loads of one key after another would each wait out the memory's latency
        constexpr int U = PIECES == 1 ? 4 : 2;
        for (int jj = 0; jj < n; jj += U * ks) {  // uniform trip count; lanes past n add nothing
          float pj[U][MAPS];
          long long off[U];
          float vv[U][PIECES][8];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int key = jj + u * ks + sub;
#pragma unroll
            for (int mm = 0; mm < MAPS; ++mm) {
              pj[u][mm] = __shfl_sync(0xffffffffu, p[mm], key & 31);
              if (key >= n) pj[u][mm] = 0.f;
            }
            off[u] = __shfl_sync(0xffffffffu, v_off, key & 31);
#pragma unroll
            for (int pc = 0; pc < PIECES; ++pc) {
              const int d0 = ((lane % lpr) + pc * lpr) * 8;
              if (key < n && d0 < VD) {
                load8<T>(vbase + off[u] + d0, vv[u][pc]);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) vv[u][pc][e] = 0.f;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int pc = 0; pc < PIECES; ++pc)
#pragma unroll
              for (int mm = 0; mm < MAPS; ++mm)
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  acc[mm][pc * 8 + e] = fmaf(pj[u][mm], vv[u][pc][e], acc[mm][pc * 8 + e]);
        }
      } else {
        for (int jj = 0; jj < n; ++jj) {
          float pj[MAPS];
#pragma unroll
          for (int mm = 0; mm < MAPS; ++mm) pj[mm] = __shfl_sync(0xffffffffu, p[mm], jj);
          const long long off = __shfl_sync(0xffffffffu, v_off, jj);
          const T* vrow = vbase + off;
#pragma unroll
          for (int i = 0; i < NACC; ++i) {
            const int d = lane + 32 * i;
            if (d < VD) {
              const float vv = fb_load_coherent<T>(vrow + d);
#pragma unroll
              for (int mm = 0; mm < MAPS; ++mm) acc[mm][i] = fmaf(pj[mm], vv, acc[mm][i]);
            }
          }
        }
      }
    }
  }
  if (VEC) {
    // the lanes that hold the same piece of the row (one per key worked at a time)
#pragma unroll
    for (int mm = 0; mm < MAPS; ++mm)
#pragma unroll
      for (int e = 0; e < NACC; ++e)
        for (int off = lpr; off < 32; off <<= 1)
          acc[mm][e] += __shfl_xor_sync(0xffffffffu, acc[mm][e], off);
  }
  // where the lane's accumulator i lies in the row, and whether this lane is the one to write it
  auto place = [&](int i) { return VEC ? ((lane % lpr) + (i / 8) * lpr) * 8 + (i % 8) : lane + 32 * i; };
  const bool writer = !VEC || lane < lpr;
  if (splits > 1) {
#pragma unroll
    for (int mm = 0; mm < MAPS; ++mm) {
      float* dst = partial + ((((size_t)t * H + a) * splits + blockIdx.z) * MAPS + mm) * (VD + 2);
      if (lane == 0) { dst[0] = m[mm]; dst[1] = l[mm]; }
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = place(i);
        if (writer && d < VD) dst[2 + d] = acc[mm][i];
      }
    }
    return;
  }
  if (MAPS == 1) {
    const float inv_l = 1.0f / l[0];
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = place(i);
      if (writer && d < VD) o[d] = fb_from_float<T>(acc[0][i] * inv_l);
    }
    return;
  }
  const float inv0 = 1.0f / l[0], inv1 = 1.0f / l[MAPS - 1];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = place(i);
    acc[0][i] = acc[0][i] * inv0 - rule.lambda * (acc[MAPS - 1][i] * inv1);
    if (writer && d < VD) ss = fmaf(acc[0][i], acc[0][i], ss);
  }
  const float r = rule.post_scale / sqrtf(fb_warp_sum(ss) / (float)VD + rule.post_eps);
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = place(i);
    if (writer && d < VD) o[d] = fb_from_float<T>(acc[0][i] * r);
  }
}

// The same attention with a chunk's 32 key rows (and value rows) staged in shared
// memory once per block: the warps of a block are query heads that share a key head
// (the heads of one token), so the rows cross from L2 once per block instead of once
// per head, in coalesced 16-byte copies; a lane then reads its key's row out of shared
// memory (rows 16 bytes longer than their data keep those reads free of bank
// conflicts). For sizes whose rows are whole 16-byte pieces. `v_in_k`: the values are
// the first VD elements of the key rows, which are staged only once.
__device__ __forceinline__ void cp_async16_s(void* dst, const void* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_all_s() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}
template <typename T>
__device__ __forceinline__ void load8s(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8s<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8s<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <typename T, int MAPS, int NACC>
__global__ void __launch_bounds__(WARPS * 32)
attention_sink_staged_kernel(const T* q, long long q_stride, T* __restrict__ out,
                             long long out_stride, const int* __restrict__ positions,
                             const int* __restrict__ seq_of_token,
                             const int* __restrict__ page_table, int max_pages, const T* k_cache,
                             const T* v_cache, long long k_page, long long k_head,
                             long long v_page, long long v_head, int k_row, int v_row,
                             ScoreRule rule, int H, int G, int D, int VD, int splits,
                             float* __restrict__ partial, int lpr, int v_in_k) {
  fb_pdl_wait();
  extern __shared__ __align__(16) unsigned char staged_smem[];
  constexpr int PIECES = NACC / 8;
  constexpr int PAD = 16 / (int)sizeof(T);
  const int KW = MAPS * D;
  const int kp = KW + PAD, vp = v_in_k ? kp : VD + PAD;  // row pitches in elements
  T* sK = reinterpret_cast<T*>(staged_smem);               // [32][kp]
  T* sV = v_in_k ? sK : sK + 32 * kp;                      // [32][vp]
  float* qs_all = reinterpret_cast<float*>(sK + 32 * kp + (v_in_k ? 0 : 32 * vp));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = qs_all + (size_t)warp * KW;
  const int t = blockIdx.x;
  const int rep = H / G;
  const int per_g = (rep + WARPS - 1) / WARPS;  // blocks that the query heads of a key head take
  const int g = blockIdx.y / per_g;
  const int within = (blockIdx.y % per_g) * WARPS + warp;
  const bool active = within < rep;             // (an idle warp still helps with the staging)
  const int a = g * rep + within;
  const int seq = seq_of_token[t];
  T* o = out + (size_t)t * out_stride + (size_t)a * VD;
  if (seq < 0) {  // padding token (the whole block): defined output, no cache access
    if (active)
      for (int d = lane; d < VD; d += 32) o[d] = fb_from_float<T>(0.f);
    return;
  }
  const int pos = positions[t];
  if (active) {
    const T* qrow = q + (size_t)t * q_stride + (size_t)a * KW;
    for (int d = lane; d < KW; d += 32) qs[d] = fb_load_coherent<T>(qrow + d);
  }
  const float slope = (active && rule.steep > 0.f) ? exp2f(-rule.steep * (float)(a + 1) / (float)H) : 0.f;
  const int lo = (rule.window > 0 && pos - rule.window + 1 > 0) ? pos - rule.window + 1 : 0;
  const int kept = min(rule.keep_first, lo);
  const int* pages = page_table + (size_t)seq * max_pages;
  const T* kbase = k_cache + (long long)g * k_head;
  const T* vbase = v_cache + (long long)g * v_head;
  const int total = kept + (pos + 1 - lo);
  const int i0 = (int)((long long)total * blockIdx.z / splits);
  const int i1 = (int)((long long)total * (blockIdx.z + 1) / splits);
  const bool own_sink = rule.sink && splits == 1;
  const float sink_score = (active && rule.sink == 2) ? rule.sink_logit[a] : 0.f;
  float m[MAPS], l[MAPS];
  float acc[MAPS][NACC];
#pragma unroll
  for (int mm = 0; mm < MAPS; ++mm) {
    m[mm] = own_sink ? sink_score : -INFINITY;
    l[mm] = own_sink ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[mm][i] = 0.f;
  }
  const int units_k = KW * (int)sizeof(T) / 16, units_v = VD * (int)sizeof(T) / 16;

  for (int range = 0; range < 2; ++range) {
    const int begin = range == 0 ? min(i0, kept) : lo + max(i0 - kept, 0);
    const int end = range == 0 ? min(i1, kept) : lo + max(i1 - kept, 0);  // exclusive
    for (int j0 = begin; j0 < end; j0 += 32) {
      const int n = min(32, end - j0);
      __syncthreads();  // the rows of the chunk before have been read by every warp
      for (int id = threadIdx.x; id < n * units_k; id += WARPS * 32) {
        const int r = id / units_k, u = id - r * units_k;
        const int j = j0 + r;
        const char* src = reinterpret_cast<const char*>(
            kbase + (long long)pages[j / FB_PAGE] * k_page + (long long)(j % FB_PAGE) * k_row);
        cp_async16_s(reinterpret_cast<char*>(sK + (size_t)r * kp) + u * 16, src + u * 16);
      }
      if (!v_in_k) {
        for (int id = threadIdx.x; id < n * units_v; id += WARPS * 32) {
          const int r = id / units_v, u = id - r * units_v;
          const int j = j0 + r;
          const char* src = reinterpret_cast<const char*>(
              vbase + (long long)pages[j / FB_PAGE] * v_page + (long long)(j % FB_PAGE) * v_row);
          cp_async16_s(reinterpret_cast<char*>(sV + (size_t)r * vp) + u * 16, src + u * 16);
        }
      }
      cp_async_all_s();
      __syncthreads();
      if (!active) continue;
      const int j = j0 + lane;
      float s[MAPS], p[MAPS];
#pragma unroll
      for (int mm = 0; mm < MAPS; ++mm) {
        s[mm] = -INFINITY;
        if (lane < n) {
          const float* qm = qs + mm * D;
          const T* km = sK + (size_t)lane * kp + mm * D;
          float d0 = 0.f, d1 = 0.f;  // two sums side by side: shorter chains
          for (int d = 0; d < D; d += 16) {
            float ka[8], kb[8], qa[8], qb[8];
            load8s<T>(km + d, ka);
            load8s<float>(qm + d, qa);  // (all lanes read the same query elements: a broadcast)
            if (d + 8 < D) {
              load8s<T>(km + d + 8, kb);
              load8s<float>(qm + d + 8, qb);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) d0 = fmaf(qa[e], ka[e], d0);
            if (d + 8 < D)
#pragma unroll
              for (int e = 0; e < 8; ++e) d1 = fmaf(qb[e], kb[e], d1);
          }
          s[mm] = capped((d0 + d1) * rule.scale, rule.softcap) - slope * (float)(pos - j);
        }
        const float m_new = fmaxf(m[mm], fb_warp_max(s[mm]));
        const float corr = expf(m[mm] - m_new);
        p[mm] = (lane < n) ? expf(s[mm] - m_new) : 0.f;
        l[mm] = l[mm] * corr + fb_warp_sum(p[mm]);
        m[mm] = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[mm][i] *= corr;
      }
      const int sub = lane / lpr, ks = 32 / lpr;
      for (int jj = 0; jj < n; jj += ks) {  // uniform trip count; lanes past n add nothing
        const int key = jj + sub;
        float pj[MAPS];
#pragma unroll
        for (int mm = 0; mm < MAPS; ++mm) pj[mm] = __shfl_sync(0xffffffffu, p[mm], key & 31);
#pragma unroll
        for (int pc = 0; pc < PIECES; ++pc) {
          const int d0 = ((lane % lpr) + pc * lpr) * 8;
          if (key < n && d0 < VD) {
            float vv[8];
            load8s<T>(sV + (size_t)key * vp + d0, vv);
#pragma unroll
            for (int mm = 0; mm < MAPS; ++mm)
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[mm][pc * 8 + e] = fmaf(pj[mm], vv[e], acc[mm][pc * 8 + e]);
          }
        }
      }
    }
  }
  if (!active) return;
#pragma unroll
  for (int mm = 0; mm < MAPS; ++mm)
#pragma unroll
    for (int e = 0; e < NACC; ++e)
      for (int off = lpr; off < 32; off <<= 1)
        acc[mm][e] += __shfl_xor_sync(0xffffffffu, acc[mm][e], off);
  auto place = [&](int i) { return ((lane % lpr) + (i / 8) * lpr) * 8 + (i % 8); };
  const bool writer = lane < lpr;
  if (splits > 1) {
#pragma unroll
    for (int mm = 0; mm < MAPS; ++mm) {
      float* dst = partial + ((((size_t)t * H + a) * splits + blockIdx.z) * MAPS + mm) * (VD + 2);
      if (lane == 0) { dst[0] = m[mm]; dst[1] = l[mm]; }
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = place(i);
        if (writer && d < VD) dst[2 + d] = acc[mm][i];
      }
    }
    return;
  }
  if (MAPS == 1) {
    const float inv_l = 1.0f / l[0];
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = place(i);
      if (writer && d < VD) o[d] = fb_from_float<T>(acc[0][i] * inv_l);
    }
    return;
  }
  const float inv0 = 1.0f / l[0], inv1 = 1.0f / l[MAPS - 1];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = place(i);
    acc[0][i] = acc[0][i] * inv0 - rule.lambda * (acc[MAPS - 1][i] * inv1);
    if (writer && d < VD) ss = fmaf(acc[0][i], acc[0][i], ss);
  }
  const float r = rule.post_scale / sqrtf(fb_warp_sum(ss) / (float)VD + rule.post_eps);
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = place(i);
    if (writer && d < VD) o[d] = fb_from_float<T>(acc[0][i] * r);
  }
}

// One warp per (token, head): the runs' partial results become the output. Lane s holds
// run s's maximum and sum (runs s and s + 32 with more than 32 runs), so the statistics
// are two loads a lane and shuffles; the runs' value rows are then summed with their
// weights, four runs' loads in flight at a time.
template <typename T, int MAPS, int NACC>
__global__ void attention_sink_merge_kernel(const float* partial, T* __restrict__ out,
                                            long long out_stride, const int* __restrict__ seq_of_token,
                                            int H, int VD, int splits, ScoreRule rule) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, a = blockIdx.y * WARPS + warp;
  if (a >= H || seq_of_token[t] < 0) return;  // padding rows were written by the first kernel
  const float sink_score = rule.sink == 2 ? rule.sink_logit[a] : 0.f;
  float acc[MAPS][NACC];
#pragma unroll
  for (int mm = 0; mm < MAPS; ++mm) {
    const float* src = partial + (((size_t)t * H + a) * splits * MAPS + mm) * (VD + 2);
    const size_t step = (size_t)MAPS * (VD + 2);  // from one run's record of this map to the next
    float ms[2], ls[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int run = lane + 32 * h;
      ms[h] = run < splits ? __ldcg(src + run * step) : -INFINITY;
      ls[h] = run < splits ? __ldcg(src + run * step + 1) : 0.f;
    }
    float M = fb_warp_max(fmaxf(ms[0], ms[1]));
    if (rule.sink) M = fmaxf(M, sink_score);
    float f[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) f[h] = ms[h] == -INFINITY ? 0.f : expf(ms[h] - M);  // 0: an empty run
    const float L = fb_warp_sum(ls[0] * f[0] + ls[1] * f[1]) + (rule.sink ? expf(sink_score - M) : 0.f);
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[mm][i] = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 4) {
      float w[4], v[4][NACC];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int run = s0 + u;
        const float both = __shfl_sync(0xffffffffu, run < 32 ? f[0] : f[1], run & 31);
        w[u] = run < splits ? both : 0.f;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
          const int d = lane + 32 * i;
          v[u][i] = (run < splits && d < VD) ? __ldcg(src + run * step + 2 + d) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[mm][i] = fmaf(v[u][i], w[u], acc[mm][i]);
    }
    const float inv = 1.0f / L;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[mm][i] *= inv;
  }
  T* o = out + (size_t)t * out_stride + (size_t)a * VD;
  float r = 1.0f;
  if (MAPS > 1) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      acc[0][i] -= rule.lambda * acc[MAPS - 1][i];
      if (lane + 32 * i < VD) ss = fmaf(acc[0][i], acc[0][i], ss);
    }
    r = rule.post_scale / sqrtf(fb_warp_sum(ss) / (float)VD + rule.post_eps);
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < VD) o[d] = fb_from_float<T>(acc[0][i] * r);
  }
}

// ------------------------------------------- queries with a temperature + cache
// q_out[t] = q[t] * (1 + coef * ln(floor((p + 1) / every) + 1)) at position p (every 0:
// the queries as they are); the token's key rows and value rows go into its cache row.
// qkv: float32 rows [q (nq) | k (G * krow) | v (G * vdim)].
template <typename T>
__global__ void q_temp_cache_kernel(const float* qkv, long long ld, T* __restrict__ q_out,
                                    float coef, int every, const int* __restrict__ positions,
                                    const int* __restrict__ seq_of_token,
                                    const int* __restrict__ page_table, int max_pages,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache,
                                    long long k_page, long long k_head, long long v_page,
                                    long long v_head, int nq, int G, int krow, int vdim,
                                    int write_cache) {
  fb_pdl_launch();
  fb_pdl_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const float* row = qkv + (size_t)t * ld;
  const int pos = seq < 0 ? 0 : positions[t];
  const float temp = every > 0 ? 1.0f + coef * logf((float)((pos + 1) / every) + 1.0f) : 1.0f;
  T* qo = q_out + (size_t)t * nq;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) qo[i] = fb_from_float<T>(__ldcg(row + i) * temp);
  if (!write_cache || seq < 0) return;
  const long long page = page_table[(size_t)seq * max_pages + pos / FB_PAGE];
  const int r = pos % FB_PAGE;
  const int nk = G * krow, nv = G * vdim;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int g = i / krow, d = i - g * krow;
    k_cache[page * k_page + g * k_head + (long long)r * krow + d] = fb_from_float<T>(__ldcg(row + nq + i));
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const int g = i / vdim, d = i - g * vdim;
    v_cache[page * v_page + g * v_head + (long long)r * vdim + d] =
        fb_from_float<T>(__ldcg(row + nq + nk + i));
  }
}

// --------------------------------------------------- latent rows: norms + rotation
// The rotation turns neighbouring pairs (2i, 2i + 1) of the first `rot_dims` elements by
// position * freq[i]; the angle is the float64 product, so it is exact to 32 bits at any position.
__device__ __forceinline__ void pair_angle(int pos, double freq, float& c, float& s) {
  double sd, cd;
  sincos((double)pos * freq, &sd, &cd);
  c = (float)cd;
  s = (float)sd;
}

// in: float32 rows [a (na) | b (nb) | rot (nrot)].
//   a_out[t] = a / sqrt(mean(a^2) + eps) * wa                      (activation type)
//   cache row of the token (one key head) = [b / sqrt(mean(b^2) + eps) * wb | rotated rot]
template <typename T>
__global__ void latent_rows_kernel(const float* in, long long ld, T* __restrict__ a_out,
                                   const float* __restrict__ wa, const float* __restrict__ wb,
                                   float eps, const double* __restrict__ freq, int rot_dims,
                                   const int* __restrict__ positions,
                                   const int* __restrict__ seq_of_token,
                                   const int* __restrict__ page_table, int max_pages,
                                   T* __restrict__ cache, long long c_page, T* __restrict__ b_out,
                                   int na, int nb, int nrot, int write_cache) {
  fb_pdl_launch();
  fb_pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const float* row = in + (size_t)t * ld;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < na; i += blockDim.x) {
    const float v = __ldcg(row + i);
    sa += v * v;
  }
  for (int i = threadIdx.x; i < nb; i += blockDim.x) {
    const float v = __ldcg(row + na + i);
    sb += v * v;
  }
  sa = fb_block_sum(sa, scratch);
  sb = fb_block_sum(sb, scratch);
  const float ra = 1.0f / sqrtf(sa / (float)na + eps);
  const float rb = 1.0f / sqrtf(sb / (float)nb + eps);
  for (int i = threadIdx.x; i < na; i += blockDim.x)
    a_out[(size_t)t * na + i] = fb_from_float<T>(__ldcg(row + i) * ra * wa[i]);
  // the same row goes to the token's place in the cache and, where asked for, to row t
  // of a buffer of the step (for a consumer that works on the step's own rows)
  const bool to_cache = write_cache && seq >= 0;
  if (!to_cache && b_out == nullptr) return;
  const int pos = seq < 0 ? 0 : positions[t];
  T* dst = !to_cache ? nullptr
      : cache + (long long)page_table[(size_t)seq * max_pages + pos / FB_PAGE] * c_page +
            (long long)(pos % FB_PAGE) * (nb + nrot);
  T* copy = b_out == nullptr ? nullptr : b_out + (size_t)t * (nb + nrot);
  auto put = [&](int i, float v) {
    const T e = fb_from_float<T>(v);
    if (dst != nullptr) dst[i] = e;
    if (copy != nullptr) copy[i] = e;
  };
  for (int i = threadIdx.x; i < nb; i += blockDim.x) put(i, __ldcg(row + na + i) * rb * wb[i]);
  const float* rot = row + na + nb;
  for (int i = threadIdx.x; i < nrot / 2 + (nrot & 1); i += blockDim.x) {
    const float u = __ldcg(rot + 2 * i);
    if (2 * i + 1 >= nrot) { put(nb + 2 * i, u); continue; }
    const float v = __ldcg(rot + 2 * i + 1);
    float c = 1.f, s = 0.f;
    if (2 * i + 1 < rot_dims) pair_angle(pos, freq[i], c, s);
    put(nb + 2 * i, u * c - v * s);
    put(nb + 2 * i + 1, v * c + u * s);
  }
}

// q: float32 rows of H heads [plain (d) | rot (c)]. The plain parts go to plain_out
// [T, H * d] (or, with `plain_into_wide`, to the first d elements of the head's wide row,
// which then is the whole rotated query head); the rotated parts, turned by the token's position, to wide_out[t, h, off : off + c]
// with rows of H * wide elements (the query rows of an attention over latent rows, whose
// first `off` elements a projection of the plain parts fills).
template <typename T>
__global__ void split_rotate_kernel(const float* q, long long ld, T* __restrict__ plain_out,
                                    T* __restrict__ wide_out, int wide, int off,
                                    const double* __restrict__ freq, int rot_dims,
                                    const int* __restrict__ positions,
                                    const int* __restrict__ seq_of_token, int H, int d, int c,
                                    int plain_into_wide) {
  fb_pdl_launch();
  fb_pdl_wait();
  extern __shared__ float cs[];  // cos, sin of the token's angles: [2][c / 2]
  const int t = blockIdx.x;
  const int pos = seq_of_token[t] < 0 ? 0 : positions[t];
  const int pairs = c / 2;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    float co = 1.f, si = 0.f;
    if (2 * i + 1 < rot_dims) pair_angle(pos, freq[i], co, si);
    cs[i] = co;
    cs[pairs + i] = si;
  }
  __syncthreads();
  const float* row = q + (size_t)t * ld;
  for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
    const int h = i / d, e = i - h * d;
    const T v = fb_from_float<T>(__ldcg(row + (size_t)h * (d + c) + e));
    if (plain_into_wide) wide_out[((size_t)t * H + h) * wide + e] = v;  // (off == d then)
    else plain_out[(size_t)t * H * d + i] = v;
  }
  for (int i = threadIdx.x; i < H * pairs; i += blockDim.x) {
    const int h = i / pairs, e = i - h * pairs;
    const float* src = row + (size_t)h * (d + c) + d + 2 * e;
    const float u = __ldcg(src), v = __ldcg(src + 1);
    T* dst = wide_out + ((size_t)t * H + h) * wide + off + 2 * e;
    dst[0] = fb_from_float<T>(u * cs[e] - v * cs[pairs + e]);
    dst[1] = fb_from_float<T>(v * cs[e] + u * cs[pairs + e]);
  }
  if (c & 1)
    for (int h = threadIdx.x; h < H; h += blockDim.x)
      wide_out[((size_t)t * H + h) * wide + off + c - 1] =
          fb_from_float<T>(__ldcg(row + (size_t)h * (d + c) + d + c - 1));
}
}  // namespace

FB_API int fb_qk_norm_cache_write(const float* qkv, long long ld, void* q_out, int dtype,
                                  const float* wq, const float* wk, float eps,
                                  const int* positions, const int* seq_of_token,
                                  const int* page_table, int max_pages, void* k_cache,
                                  void* v_cache, long long k_page, long long k_head,
                                  long long v_page, long long v_head, int T, int H, int G, int dim,
                                  int vdim, int write_cache, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && G > 0 && dim > 0 && vdim > 0, "qk_norm_cache_write: bad sizes");
  FB_REQUIRE(ld >= (long long)H * dim + (long long)G * (dim + vdim),
             "qk_norm_cache_write: rows of %lld hold no q, k and v", ld);
  FB_REQUIRE(!write_cache || (k_cache && v_cache && page_table && max_pages > 0),
             "qk_norm_cache_write: no cache to write");
  if (T == 0) return 0;
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(qk_norm_cache_kernel<E>, dim3(T), dim3(256), 0, stream,
      qkv, ld, (E*)q_out, wq, wk, eps, positions, seq_of_token, page_table, max_pages,
      (E*)k_cache, (E*)v_cache, k_page, k_head, v_page, v_head, H, G, dim, vdim, write_cache)));
  return fb_check_launch("qk_norm_cache_write");
}

FB_API int fb_q_temp_cache_write(const float* qkv, long long ld, void* q_out, int dtype,
                                 float coef, int every, const int* positions,
                                 const int* seq_of_token, const int* page_table, int max_pages,
                                 void* k_cache, void* v_cache, long long k_page, long long k_head,
                                 long long v_page, long long v_head, int T, int nq, int G, int krow,
                                 int vdim, int write_cache, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && nq > 0 && G > 0 && krow > 0 && vdim > 0 && every >= 0,
             "q_temp_cache_write: bad sizes");
  FB_REQUIRE(ld >= (long long)nq + (long long)G * (krow + vdim),
             "q_temp_cache_write: rows of %lld hold no q, k and v", ld);
  FB_REQUIRE(!write_cache || (k_cache && v_cache && page_table && max_pages > 0),
             "q_temp_cache_write: no cache to write");
  if (T == 0) return 0;
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(q_temp_cache_kernel<E>, dim3(T), dim3(256), 0, stream,
      qkv, ld, (E*)q_out, coef, every, positions, seq_of_token, page_table, max_pages,
      (E*)k_cache, (E*)v_cache, k_page, k_head, v_page, v_head, nq, G, krow, vdim, write_cache)));
  return fb_check_launch("q_temp_cache_write");
}

FB_API int fb_latent_rows(const float* in, long long ld, void* a_out, int dtype, const float* wa,
                          const float* wb, float eps, const double* freq, int rot_dims,
                          const int* positions, const int* seq_of_token, const int* page_table,
                          int max_pages, void* cache, long long c_page, void* b_out, int T, int na,
                          int nb, int nrot, int write_cache, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && na >= 0 && nb > 0 && nrot >= 0 && rot_dims >= 0 && rot_dims <= nrot &&
             rot_dims % 2 == 0, "latent_rows: bad sizes");  // na = 0: no second latent
  FB_REQUIRE(ld >= (long long)na + nb + nrot, "latent_rows: rows of %lld are too short", ld);
  FB_REQUIRE(!write_cache || (cache && page_table && max_pages > 0), "latent_rows: no cache to write");
  if (T == 0) return 0;
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(latent_rows_kernel<E>, dim3(T), dim3(256), 0, stream, in,
      ld, (E*)a_out, wa, wb, eps, freq, rot_dims, positions, seq_of_token, page_table, max_pages,
      (E*)cache, c_page, (E*)b_out, na, nb, nrot, write_cache)));
  return fb_check_launch("latent_rows");
}

FB_API int fb_split_rotate(const float* q, long long ld, void* plain_out, void* wide_out, int dtype,
                           int wide, int off, const double* freq, int rot_dims,
                           const int* positions, const int* seq_of_token, int T, int H, int d,
                           int c, int plain_into_wide, cudaStream_t stream) {
  FB_REQUIRE(plain_into_wide ? off == d : plain_out != nullptr,
             "split_rotate: the plain parts have no place");
  FB_REQUIRE(T >= 0 && H > 0 && d > 0 && c >= 0 && off >= 0 && off + c <= wide &&
             rot_dims >= 0 && rot_dims <= c && rot_dims % 2 == 0, "split_rotate: bad sizes");
  FB_REQUIRE(ld >= (long long)H * (d + c), "split_rotate: rows of %lld are too short", ld);
  if (T == 0) return 0;
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(split_rotate_kernel<E>, dim3(T), dim3(256),
      (size_t)(c / 2 * 2 + 2) * 4, stream, q, ld, (E*)plain_out, (E*)wide_out, wide, off, freq,
      rot_dims, positions, seq_of_token, H, d, c, plain_into_wide)));
  return fb_check_launch("split_rotate");
}

FB_API int fb_attention_sink(const void* q, long long q_stride, void* out, long long out_stride,
                             int dtype, const int* positions, const int* seq_of_token,
                             const int* page_table, int max_pages, const void* k_cache,
                             const void* v_cache, long long k_page, long long k_head,
                             long long v_page, long long v_head, int k_row, int v_row, int window,
                             int keep_first, int sink, const float* sink_logit, float scale,
                             float steep, float softcap, int maps, float lambda, float post_eps,
                             float post_scale, int T, int H, int G, int D, int VD, int splits,
                             float* partial, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && G > 0 && D > 0 && VD > 0, "attention_sink: bad sizes");
  FB_REQUIRE(H % G == 0, "attention_sink: %d query heads are not a multiple of %d key-value heads",
             H, G);
  FB_REQUIRE(maps == 1 || maps == 2, "attention_sink: %d maps a head (1 or 2)", maps);
  FB_REQUIRE(maps * D <= MAX_QD && VD <= (maps == 1 ? 768 : 256),
             "attention_sink: key size %d x %d maps and value size %d are beyond the kernel's %d "
             "and %d", D, maps, VD, MAX_QD, maps == 1 ? 768 : 256);
  FB_REQUIRE(k_row >= maps * D && v_row >= 1, "attention_sink: rows shorter than their vectors");
  FB_REQUIRE(sink >= 0 && sink <= 2 && (sink != 2 || sink_logit != nullptr),
             "attention_sink: a sink with a score per head needs the scores");
  const int kvec = D % 8 == 0 && k_row % 8 == 0 && k_page % 8 == 0 && k_head % 8 == 0 &&
                   ((uintptr_t)k_cache % 32) == 0;
  FB_REQUIRE(window >= 0 && keep_first >= 0 && max_pages > 0, "attention_sink: bad mask");
  FB_REQUIRE(splits >= 1 && splits <= 64 && (splits == 1 || partial != nullptr),
             "attention_sink: %d runs need a workspace", splits);
  if (T == 0) return 0;
  ScoreRule rule{window, keep_first, sink, sink_logit, scale, steep, softcap, lambda, post_eps,
                 post_scale};
  dim3 grid(T, (H + WARPS - 1) / WARPS, splits);
  const bool vec = VD % 8 == 0 && v_row % 8 == 0 && v_page % 8 == 0 && v_head % 8 == 0 &&
                   ((uintptr_t)v_cache % 32) == 0;
  int lpr = 1;
  while (lpr * 8 < VD && lpr < 32) lpr *= 2;  // lanes that share a value row: a power of two
  const size_t smem = (size_t)WARPS * maps * D * 4;
  const bool wide = VD > 256;
  // Rows of whole 16-byte pieces: the form that stages a chunk's rows in shared memory
  // once for the query heads of a key head.
  const int v_in_k = v_cache == k_cache && v_row == k_row && v_page == k_page && v_head == k_head;
  const int elt = dtype == FB_F32 ? 4 : 2, pad = 16 / elt;
  const size_t staged_smem = (size_t)32 * (maps * D + pad) * elt +
                             (v_in_k ? 0 : (size_t)32 * (VD + pad) * elt) +
                             (size_t)WARPS * maps * D * 4;
  if (vec && kvec && v_row % 8 == 0 && staged_smem <= 160 * 1024) {
    const int rep = H / G;
    dim3 sgrid(T, G * ((rep + WARPS - 1) / WARPS), splits);
#define FB_STAGED_LAUNCH(MAPS_, NACC_)                                                          \
    FB_DISPATCH_DTYPE(dtype, E, {                                                               \
      static bool seen[64];                                                                     \
      if (staged_smem > 48 * 1024 && fb_first_use_on_device(seen))                              \
        cudaFuncSetAttribute(attention_sink_staged_kernel<E, MAPS_, NACC_>,                     \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);          \
      fb_launch(attention_sink_staged_kernel<E, MAPS_, NACC_>, dim3(sgrid), dim3(WARPS * 32),   \
          staged_smem, stream, (const E*)q, q_stride, (E*)out, out_stride, positions,           \
          seq_of_token, page_table, max_pages, (const E*)k_cache, (const E*)v_cache, k_page,    \
          k_head, v_page, v_head, k_row, v_row, rule, H, G, D, VD, splits, partial, lpr,        \
          v_in_k); })
    if (maps == 2) FB_STAGED_LAUNCH(2, 8);
    else if (wide) FB_STAGED_LAUNCH(1, 24);
    else FB_STAGED_LAUNCH(1, 8);
#undef FB_STAGED_LAUNCH
  } else {
#define FB_SINK_LAUNCH(VEC_, MAPS_, NACC_)                                                       \
  FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_sink_kernel<E, VEC_, MAPS_, NACC_>,          \
      dim3(grid), dim3(WARPS * 32), smem, stream, (const E*)q, q_stride, (E*)out, out_stride,    \
      positions, seq_of_token, page_table, max_pages, (const E*)k_cache, (const E*)v_cache,      \
      k_page, k_head, v_page, v_head, k_row, v_row, rule, H, G, D, VD, splits, partial, lpr,     \
      kvec)))
  if (maps == 2) { if (vec) FB_SINK_LAUNCH(true, 2, 8); else FB_SINK_LAUNCH(false, 2, 8); }
  else if (wide) { if (vec) FB_SINK_LAUNCH(true, 1, 24); else FB_SINK_LAUNCH(false, 1, 24); }
  else { if (vec) FB_SINK_LAUNCH(true, 1, 8); else FB_SINK_LAUNCH(false, 1, 8); }
#undef FB_SINK_LAUNCH
  }
  if (splits > 1) {
    int rc = fb_check_launch("attention_sink");
    if (rc) return rc;
#define FB_MERGE_LAUNCH(MAPS_, NACC_)                                                          \
    FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_sink_merge_kernel<E, MAPS_, NACC_>,      \
        dim3(T, (H + WARPS - 1) / WARPS), dim3(WARPS * 32), 0, stream, (const float*)partial,  \
        (E*)out, out_stride, seq_of_token, H, VD, splits, rule)))
    if (maps == 2) FB_MERGE_LAUNCH(2, 8);
    else if (wide) FB_MERGE_LAUNCH(1, 24);
    else FB_MERGE_LAUNCH(1, 8);
#undef FB_MERGE_LAUNCH
  }
  return fb_check_launch("attention_sink");
}

// The merge alone, for a kernel of another file that leaves the same records: partial
// [T * H, splits, VD + 2] of (max, sum, weighted values), one map; bfloat16 or float32 out.
FB_API int fb_attention_sink_merge(const float* partial, void* out, long long out_stride, int dtype,
                                   const int* seq_of_token, int T, int H, int VD, int splits,
                                   const float* sink_logit, cudaStream_t stream) {
  FB_REQUIRE(T >= 0 && H > 0 && VD > 0 && VD <= 768 && splits >= 1 && splits <= 64 && partial != nullptr,
             "attention_sink_merge: bad sizes");
  if (T == 0) return 0;
  ScoreRule rule{0, 0, sink_logit != nullptr ? 2 : 0, sink_logit, 1.f, 0.f, 0.f, 0.f, 0.f, 1.f};
  if (VD > 256) {
    FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_sink_merge_kernel<E, 1, 24>,
        dim3(T, (H + WARPS - 1) / WARPS), dim3(WARPS * 32), 0, stream, partial, (E*)out, out_stride,
        seq_of_token, H, VD, splits, rule)));
  } else {
    FB_DISPATCH_DTYPE(dtype, E, (fb_launch(attention_sink_merge_kernel<E, 1, 8>,
        dim3(T, (H + WARPS - 1) / WARPS), dim3(WARPS * 32), 0, stream, partial, (E*)out, out_stride,
        seq_of_token, H, VD, splits, rule)));
  }
  return fb_check_launch("attention_sink_merge");
}
