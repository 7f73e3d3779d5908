// bfloat16 prompt attention on the tensor cores for heads whose keys and values
// have different sizes, with a score cap, a learned sink, and two maps a head.
//
//   s = cap(q . k * scale),  cap(x) = softcap * tanh(x / softcap)  (softcap 0: x);  causal
//   one map:   p = exp(s) / (exp(sink_h) + sum exp(s))   (no sink: the plain softmax);  o = sum p v
//   two maps:  a query head has two query vectors and a key row two key vectors of DK side by
//              side; each map is a softmax attention of its own over the same value rows, and
//              o = a1 - lambda a2;  o <- o / sqrt(mean(o^2) + eps) * post_scale
//
// A 64-row block of one sequence's queries for one head walks the sequence's keys 64 at
// a time with an online softmax (log2 domain); the four warps own 16 query rows each;
// mma.sync.m16n8k16 with 32-bit accumulation, probabilities rounded to bfloat16 only as
// the operand of the P.V product. With two maps both score tiles are made from one key
// tile and every value fragment is loaded once for both.
//
// Keys and values come from one of two places: the paged cache (a key row of
// MAPS * DK elements per key head, value rows of DV in a storage of their own), or rows
// of the step's own tokens (`paged` 0: for steps in which every sequence begins at its
// first token, so that all keys are the step's), where a key row may be put together
// from two sources (the first K1 elements per head from one buffer, the rest, shared by
// all heads, from another).
#include "common.cuh"
#include "mma_tiles.cuh"

namespace {

using namespace fb_mma;

struct MapsParams {
  const __nv_bfloat16* q; long long q_stride;   // head h at h * MAPS * DK
  __nv_bfloat16* out; long long out_stride;     // head h at h * DV
  const int* cu_tokens;  // [n_seqs + 1]
  const int* kv_lens;    // [n_seqs]: length after this step
  const int* page_table; int max_pages;
  const __nv_bfloat16* k;   // paged: the key cache; rows: the first K1 elements of a key, per head
  const __nv_bfloat16* k2;  // rows: the other DK - K1 elements, shared by all heads (or null)
  const __nv_bfloat16* v;
  long long k_page, k_head, v_page, v_head;  // paged: page and key-head strides; rows: head offsets
  long long k_row, k2_row, v_row;            // elements from one key's row to the next
  int paged, K1;
  int n_seqs, H, G;
  float scale, softcap;
  const float* sink_logit;  // [H] or null
  float lambda, post_eps, post_scale;
};

template <int DK, int DV, int MAPS>
__global__ void __launch_bounds__(THREADS) attn_maps_kernel(const MapsParams p) {
  fb_pdl_wait();
  constexpr int KW = MAPS * DK;          // elements of a key row and of a query head
  constexpr int PK = pitch_of(KW), PV = pitch_of(DV);
  constexpr int KT = DK / 16;            // k-steps of Q.K^T per map
  constexpr int NT = DV / 8;             // n-tiles of P.V
  extern __shared__ __align__(128) uint8_t smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* sK = sQ + 64 * PK;      // [2][64][PK]
  __nv_bfloat16* sV = sK + 2 * 64 * PK;  // [2][64][PV]
  __shared__ int s_info[2];

  if (threadIdx.x == 0) {
    // Later blocks of a sequence walk more keys: hand them out first.
    int b = (int)(gridDim.x - 1 - blockIdx.x), s = 0;
    for (; s < p.n_seqs; ++s) {
      const int nb = (p.cu_tokens[s + 1] - p.cu_tokens[s] + 63) / 64;
      if (b < nb) break;
      b -= nb;
    }
    s_info[0] = s < p.n_seqs ? s : -1;
    s_info[1] = b;
  }
  __syncthreads();
  const int seq = s_info[0];
  if (seq < 0) return;
  const int row0 = s_info[1] * 64;
  const int head = blockIdx.y, kvh = head / (p.H / p.G);
  const int tok0 = p.cu_tokens[seq], q_len = p.cu_tokens[seq + 1] - tok0;
  const int kv_len = p.kv_lens[seq];
  const int pos0 = kv_len - q_len + row0;  // position of this block's first query
  const int rows_valid = min(64, q_len - row0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int last_key = pos0 + rows_valid - 1;
  const int n_pages = last_key / FB_PAGE + 1;
  const int* pages = p.page_table + (size_t)seq * p.max_pages;

  auto load_kv = [&](int stage, int pg) {
    __nv_bfloat16* dK = sK + stage * 64 * PK;
    __nv_bfloat16* dV = sV + stage * 64 * PV;
    if (p.paged) {
      const long long page = pages[pg];
      load_cols<PK>(dK, p.k + page * p.k_page + kvh * p.k_head, p.k_row, 64, 64, KW, 0);
      load_cols<PV>(dV, p.v + page * p.v_page + kvh * p.v_head, p.v_row, 64, 64, DV, 0);
    } else {
      const long long first = tok0 + (long long)pg * 64;   // (pos0 counts from 0 here)
      const int valid = min(64, kv_len - pg * 64);
      load_cols<PK>(dK, p.k + first * p.k_row + kvh * p.k_head, p.k_row, 64, valid, p.K1, 0);
      if (p.K1 < KW)
        load_cols<PK>(dK, p.k2 + first * p.k2_row, p.k2_row, 64, valid, KW - p.K1, p.K1);
      load_cols<PV>(dV, p.v + first * p.v_row + kvh * p.v_head, p.v_row, 64, valid, DV, 0);
    }
  };

  load_cols<PK>(sQ, p.q + (long long)(tok0 + row0) * p.q_stride + (long long)head * KW, p.q_stride,
                64, rows_valid, KW, 0);
  load_kv(0, 0);
  cp_async_commit();

  uint32_t qf[MAPS][KT][4];
  float o[MAPS][NT][4];
  float m[MAPS][2], l[MAPS][2];
  const float sink2 = p.sink_logit != nullptr ? p.sink_logit[head] * LOG2E : 0.f;
#pragma unroll
  for (int mm = 0; mm < MAPS; ++mm) {
#pragma unroll
    for (int n = 0; n < NT; ++n) o[mm][n][0] = o[mm][n][1] = o[mm][n][2] = o[mm][n][3] = 0.f;
    m[mm][0] = m[mm][1] = p.sink_logit != nullptr ? sink2 : -INFINITY;  // the sink: one more term
    l[mm][0] = l[mm][1] = p.sink_logit != nullptr ? 1.f : 0.f;
  }
  const int qpos_lo = pos0 + warp * 16 + g;  // position of row g; row g + 8 is 8 further
  const float inv_cap = p.softcap > 0.f ? 1.0f / p.softcap : 0.f;

  for (int pg = 0; pg < n_pages; ++pg) {
    const int st = pg & 1;
    if (pg + 1 < n_pages) load_kv(st ^ 1, pg + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (pg == 0) {
#pragma unroll
      for (int mm = 0; mm < MAPS; ++mm)
#pragma unroll
        for (int k = 0; k < KT; ++k)
          ldsm_x4(qf[mm][k], smem_u32(sQ + Swz<PK>::off(warp * 16 + (lane & 15),
                                                        mm * DK + k * 16 + (lane >> 4) * 8)));
    }
    const int key0 = pg * FB_PAGE;
    if (key0 <= pos0 + warp * 16 + 15) {  // else every query of the warp lies before these keys
      const __nv_bfloat16* tK = sK + st * 64 * PK;
      const __nv_bfloat16* tV = sV + st * 64 * PV;
      const bool need_mask = key0 + FB_PAGE - 1 > pos0 + warp * 16;
      uint32_t pa[MAPS][4][4];  // the probabilities as A operands: [map][16 keys][fragment]
#pragma unroll
      for (int mm = 0; mm < MAPS; ++mm) {
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KT; ++k) {
#pragma unroll
          for (int n2 = 0; n2 < 4; ++n2) {  // two n-tiles (16 keys) per ldmatrix.x4
            uint32_t b[4];
            ldsm_x4(b, smem_u32(tK + Swz<PK>::off(n2 * 16 + (lane & 7) + (lane >> 4) * 8,
                                                  mm * DK + k * 16 + ((lane >> 3) & 1) * 8)));
            mma_bf16(s[2 * n2], qf[mm][k], b[0], b[1]);
            mma_bf16(s[2 * n2 + 1], qf[mm][k], b[2], b[3]);
          }
        }
        float mx[2] = {m[mm][0], m[mm][1]};
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float v = s[n][e] * p.scale;
            if (p.softcap > 0.f) {
              // cap * tanh(v / cap) with tanh(x) = 1 - 2 / (exp(2x) + 1)
              const float ex = exp2f(2.0f * LOG2E * v * inv_cap);
              v = p.softcap * (1.0f - __fdividef(2.0f, ex + 1.0f));
            }
            v *= LOG2E;
            if (need_mask) {
              const int key = key0 + n * 8 + 2 * t + (e & 1);
              if (key > qpos_lo + (e >> 1) * 8) v = -INFINITY;
            }
            s[n][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
          }
        }
        float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
          corr[r] = exp2f(m[mm][r] - mx[r]);  // 0 on the first keys without a sink
          // (padding rows of the block may see no key: nothing to rescale)
          if (mx[r] == -INFINITY) { corr[r] = 1.f; mx[r] = 0.f; }
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float pv = exp2f(s[n][e] - mx[e >> 1]);
            s[n][e] = pv;
            sum[e >> 1] += pv;
          }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
          sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
          l[mm][r] = l[mm][r] * corr[r] + sum[r];
          m[mm][r] = (sum[r] == 0.f && l[mm][r] == 0.f) ? -INFINITY : mx[r];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          o[mm][n][0] *= corr[0]; o[mm][n][1] *= corr[0];
          o[mm][n][2] *= corr[1]; o[mm][n][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          pa[mm][kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
          pa[mm][kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
          pa[mm][kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
          pa[mm][kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        }
      }
      // O += P V for every map: a value fragment is loaded once
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int n2 = 0; n2 < NT / 2; ++n2) {
          uint32_t b[4];
          ldsm_x4_trans(b, smem_u32(tV + Swz<PV>::off(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                     n2 * 16 + (lane >> 4) * 8)));
#pragma unroll
          for (int mm = 0; mm < MAPS; ++mm) {
            mma_bf16(o[mm][2 * n2], pa[mm][kk], b[0], b[1]);
            mma_bf16(o[mm][2 * n2 + 1], pa[mm][kk], b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();  // the stage is refilled two iterations on
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + r * 8;
    const float inv0 = 1.0f / l[0][r];
    float mul = inv0;
    if (MAPS == 2) {
      const float inv1 = 1.0f / l[MAPS - 1][r];
      float ss = 0.f;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float v = o[0][n][2 * r + e] * inv0 - p.lambda * (o[MAPS - 1][n][2 * r + e] * inv1);
          o[0][n][2 * r + e] = v;
          ss = fmaf(v, v, ss);
        }
      }
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      mul = p.post_scale / sqrtf(ss / (float)DV + p.post_eps);
    }
    if (row < rows_valid) {
      __nv_bfloat16* dst = p.out + (long long)(tok0 + row0 + row) * p.out_stride + (long long)head * DV;
#pragma unroll
      for (int n = 0; n < NT; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) =
            pack_bf16(o[0][n][2 * r] * mul, o[0][n][2 * r + 1] * mul);
    }
  }
}

// ------------------------------------------------- heads as rows over shared key rows
// Attention of ALL query heads over one key row per token whose first DV_ALL elements are
// also the value (the folded form of a latent attention: query rows of KW = DV_ALL + rotated
// elements). The 64 rows of a block are consecutive (token, head) pairs of one sequence, so a
// token's heads share every key tile: row R of the sequence's rows is head R % H of its token
// R / H, at that token's position. A block makes DVC of the value columns (blockIdx.y picks
// which), and with `splits` > 1 walks only its share of the pages and leaves (max, sum,
// weighted values) for the merge kernel of csrc/sink_attention.cu (natural-log maxima), which
// also adds the sink; unsplit, the sink is the start of the running maximum and sum.
// The query fragments are read from shared memory at every k-step (a block's registers hold
// the 64 x DVC output), the key tile's pitch P is KW rounded up to 64 elements.
struct FoldedParams {
  const __nv_bfloat16* q;    // [rows, KW]: row (token * H + head)
  __nv_bfloat16* out;        // [rows, DV_ALL]
  float* partial;            // [rows, splits, DV_ALL + 2] or null
  const int* cu_tokens; const int* kv_lens; const int* page_table; int max_pages;
  const __nv_bfloat16* k; long long k_page;   // the cache: [pages, 1, 64, KW]
  int n_seqs, H, KW, DV_ALL, splits;
  float scale;
  const float* sink_logit;   // [H] or null
};

template <int P, int DVC>
__global__ void __launch_bounds__(THREADS) attn_folded_kernel(const FoldedParams p) {
  fb_pdl_wait();
  constexpr int NT = DVC / 8;
  extern __shared__ __align__(128) uint8_t smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* sK = sQ + 64 * P;  // [2][64][P]
  __shared__ int s_info[2];
  if (threadIdx.x == 0) {
    int b = (int)(gridDim.x - 1 - blockIdx.x), s = 0;
    for (; s < p.n_seqs; ++s) {
      const int nb = ((p.cu_tokens[s + 1] - p.cu_tokens[s]) * p.H + 63) / 64;
      if (b < nb) break;
      b -= nb;
    }
    s_info[0] = s < p.n_seqs ? s : -1;
    s_info[1] = b;
  }
  __syncthreads();
  const int seq = s_info[0];
  if (seq < 0) return;
  const int H = p.H, KW = p.KW;
  const int row0 = s_info[1] * 64;
  const int tok0 = p.cu_tokens[seq], q_len = p.cu_tokens[seq + 1] - tok0;
  const int kv_len = p.kv_lens[seq];
  const int pos_first = kv_len - q_len;
  const int rows_valid = min(64, q_len * H - row0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int vcol0 = blockIdx.y * DVC;
  const int last_pos = pos_first + (row0 + rows_valid - 1) / H;
  const int n_pages = last_pos / FB_PAGE + 1;
  const int pg0 = (int)((long long)n_pages * blockIdx.z / p.splits);
  const int pg1 = (int)((long long)n_pages * (blockIdx.z + 1) / p.splits);
  const int* pages = p.page_table + (size_t)seq * p.max_pages;
  const long long grow0 = (long long)tok0 * H + row0;  // the block's first row among all rows

  load_cols<P>(sQ, p.q + grow0 * KW, KW, 64, rows_valid, KW, 0);
  if (pg0 < pg1) load_cols<P>(sK, p.k + (long long)pages[pg0] * p.k_page, KW, 64, 64, KW, 0);
  cp_async_commit();

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m[2], l[2];
  int qpos[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + warp * 16 + g + r * 8;
    qpos[r] = pos_first + row / H;
    const bool own_sink = p.sink_logit != nullptr && p.splits == 1;
    m[r] = own_sink ? p.sink_logit[row % H] * LOG2E : -INFINITY;
    l[r] = own_sink ? 1.f : 0.f;
  }
  const float scale2 = p.scale * LOG2E;
  const int first_pos_warp = pos_first + (row0 + warp * 16) / H;
  const int last_pos_warp = pos_first + (row0 + warp * 16 + 15) / H;

  for (int pg = pg0; pg < pg1; ++pg) {
    const int st = (pg - pg0) & 1;
    if (pg + 1 < pg1)
      load_cols<P>(sK + (st ^ 1) * 64 * P, p.k + (long long)pages[pg + 1] * p.k_page, KW, 64, 64, KW, 0);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int key0 = pg * FB_PAGE;
    if (key0 <= last_pos_warp) {
      const __nv_bfloat16* tK = sK + st * 64 * P;
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      for (int k = 0; k < KW / 16; ++k) {
        uint32_t qf[4];
        ldsm_x4(qf, smem_u32(sQ + Swz<P>::off(warp * 16 + (lane & 15), k * 16 + (lane >> 4) * 8)));
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {
          uint32_t b[4];
          ldsm_x4(b, smem_u32(tK + Swz<P>::off(n2 * 16 + (lane & 7) + (lane >> 4) * 8,
                                                k * 16 + ((lane >> 3) & 1) * 8)));
          mma_bf16(s[2 * n2], qf, b[0], b[1]);
          mma_bf16(s[2 * n2 + 1], qf, b[2], b[3]);
        }
      }
      const bool need_mask = key0 + FB_PAGE - 1 > first_pos_warp;
      float mx[2] = {m[0], m[1]};
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[n][e] * scale2;
          if (need_mask && key0 + n * 8 + 2 * t + (e & 1) > qpos[e >> 1]) v = -INFINITY;
          s[n][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        corr[r] = exp2f(m[r] - mx[r]);
        if (mx[r] == -INFINITY) { corr[r] = 1.f; mx[r] = 0.f; }  // nothing seen yet
      }
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[n][e] - mx[e >> 1]);
          s[n][e] = pv;
          sum[e >> 1] += pv;
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        l[r] = l[r] * corr[r] + sum[r];
        m[r] = (sum[r] == 0.f && l[r] == 0.f) ? -INFINITY : mx[r];
      }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0];
        o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int n2 = 0; n2 < NT / 2; ++n2) {
          uint32_t b[4];
          ldsm_x4_trans(b, smem_u32(tK + Swz<P>::off(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                    vcol0 + n2 * 16 + (lane >> 4) * 8)));
          mma_bf16(o[2 * n2], a, b[0], b[1]);
          mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();  // (a block without pages has only asked for its queries)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + r * 8;
    if (row >= rows_valid) continue;
    if (p.splits > 1) {
      float* dst = p.partial + ((grow0 + row) * p.splits + blockIdx.z) * (p.DV_ALL + 2);
      if (t == 0 && blockIdx.y == 0) { dst[0] = m[r] / LOG2E; dst[1] = l[r]; }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        dst[2 + vcol0 + n * 8 + 2 * t] = o[n][2 * r];
        dst[2 + vcol0 + n * 8 + 2 * t + 1] = o[n][2 * r + 1];
      }
    } else {
      const float inv = 1.0f / l[r];
      __nv_bfloat16* dst = p.out + (grow0 + row) * p.DV_ALL + vcol0;
#pragma unroll
      for (int n = 0; n < NT; ++n)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = pack_bf16(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
    }
  }
}

template <int P, int DVC>
int launch_folded(const FoldedParams& p, int q_blocks, cudaStream_t stream) {
  const size_t smem = (size_t)3 * 64 * P * sizeof(__nv_bfloat16);
  static bool seen[64];
  if (smem > 48 * 1024 && fb_first_use_on_device(seen))
    cudaFuncSetAttribute(attn_folded_kernel<P, DVC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  fb_launch(attn_folded_kernel<P, DVC>, dim3(q_blocks, p.DV_ALL / DVC, p.splits), dim3(THREADS), smem,
            stream, p);
  return fb_check_launch("attention_folded");
}

template <int DK, int DV, int MAPS>
int launch_maps(const MapsParams& p, int q_blocks, cudaStream_t stream) {
  constexpr int PK = pitch_of(MAPS * DK), PV = pitch_of(DV);
  const size_t smem = (size_t)(3 * 64 * PK + 2 * 64 * PV) * sizeof(__nv_bfloat16);
  static bool seen[64];
  if (smem > 48 * 1024 && fb_first_use_on_device(seen))
    cudaFuncSetAttribute(attn_maps_kernel<DK, DV, MAPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
  fb_launch(attn_maps_kernel<DK, DV, MAPS>, dim3(q_blocks, p.H), dim3(THREADS), smem, stream, p);
  return fb_check_launch("attention_maps");
}
}  // namespace

// Whether a (key size per map, value size, maps) combination has a kernel here.
FB_API int fb_attention_maps_fits(int DK, int DV, int maps) {
  if (maps == 2)
    return (DK == 16 && DV == 32) || (DK == 32 && (DV == 32 || DV == 64)) ||
           (DK == 64 && (DV == 64 || DV == 128));
  return (DK == 48 && DV == 16) || (DK == 48 && DV == 32) || (DK == 80 && DV == 64) ||
         (DK == 96 && DV == 64) || (DK == 192 && DV == 128);
}

FB_API int fb_attention_maps(const void* q, long long q_stride, void* out, long long out_stride,
                             const int* cu_tokens, const int* kv_lens, const int* page_table,
                             int max_pages, const void* k, const void* k2, const void* v,
                             long long k_page, long long k_head, long long v_page, long long v_head,
                             long long k_row, long long k2_row, long long v_row, int paged, int K1,
                             int n_seqs, int q_blocks, int H, int G, int DK, int DV, int maps,
                             float scale, float softcap, const float* sink_logit, float lambda,
                             float post_eps, float post_scale, cudaStream_t stream) {
  FB_REQUIRE(n_seqs >= 0 && q_blocks >= 0 && H > 0 && G > 0 && H % G == 0, "attention_maps: bad sizes");
  FB_REQUIRE(fb_attention_maps_fits(DK, DV, maps),
             "attention_maps: no kernel for keys of %d, values of %d and %d maps", DK, DV, maps);
  const int KW = maps * DK;
  FB_REQUIRE(paged ? (page_table != nullptr && max_pages > 0 && K1 == KW)
                   : (K1 > 0 && K1 <= KW && K1 % 8 == 0 && (K1 == KW || k2 != nullptr)),
             "attention_maps: the keys' source does not fit");
  FB_REQUIRE(((uintptr_t)q | (uintptr_t)k | (uintptr_t)k2 | (uintptr_t)v | (uintptr_t)out) % 16 == 0 &&
             q_stride % 8 == 0 && out_stride % 2 == 0 && k_row % 8 == 0 && k2_row % 8 == 0 &&
             v_row % 8 == 0 && k_page % 8 == 0 && k_head % 8 == 0 && v_page % 8 == 0 && v_head % 8 == 0,
             "attention_maps: rows must start on 16-byte boundaries");
  if (n_seqs == 0 || q_blocks == 0) return 0;
  MapsParams p{(const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, cu_tokens,
               kv_lens, page_table, max_pages, (const __nv_bfloat16*)k, (const __nv_bfloat16*)k2,
               (const __nv_bfloat16*)v, k_page, k_head, v_page, v_head, k_row, k2_row, v_row,
               paged, K1, n_seqs, H, G, scale, softcap, sink_logit, lambda, post_eps, post_scale};
#define FB_MAPS(DK_, DV_, M_) \
  if (DK == DK_ && DV == DV_ && maps == M_) return launch_maps<DK_, DV_, M_>(p, q_blocks, stream)
  FB_MAPS(16, 32, 2); FB_MAPS(32, 32, 2); FB_MAPS(32, 64, 2); FB_MAPS(64, 64, 2); FB_MAPS(64, 128, 2);
  FB_MAPS(48, 16, 1); FB_MAPS(48, 32, 1); FB_MAPS(80, 64, 1); FB_MAPS(96, 64, 1); FB_MAPS(192, 128, 1);
#undef FB_MAPS
  return fb_fail(1, "attention_maps: no kernel");
}

// The folded latent attention on the tensor cores (see `attn_folded_kernel`). KW and DV:
// (144, 128), (288, 256), (576, 512). `partial` with splits > 1; the caller then runs the merge.
FB_API int fb_attention_folded(const void* q, void* out, float* partial, const int* cu_tokens,
                               const int* kv_lens, const int* page_table, int max_pages,
                               const void* k_cache, long long k_page, int n_seqs, int q_blocks,
                               int H, int KW, int DV, int splits, float scale,
                               const float* sink_logit, cudaStream_t stream) {
  FB_REQUIRE(n_seqs >= 0 && q_blocks >= 0 && H > 0 && splits >= 1 && splits <= 64 &&
             (splits == 1 || partial != nullptr), "attention_folded: bad sizes");
  FB_REQUIRE((KW == 144 && DV == 128) || (KW == 288 && DV == 256) || (KW == 576 && DV == 512),
             "attention_folded: no kernel for key rows of %d with values of %d", KW, DV);
  FB_REQUIRE(((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)out) % 16 == 0 && k_page % 8 == 0 &&
             page_table != nullptr && max_pages > 0, "attention_folded: rows must start on 16-byte boundaries");
  if (n_seqs == 0 || q_blocks == 0) return 0;
  FoldedParams p{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, partial, cu_tokens, kv_lens, page_table,
                 max_pages, (const __nv_bfloat16*)k_cache, k_page, n_seqs, H, KW, DV, splits, scale,
                 sink_logit};
  if (KW == 144) return launch_folded<192, 128>(p, q_blocks, stream);
  if (KW == 288) return launch_folded<320, 256>(p, q_blocks, stream);
  return launch_folded<576, 256>(p, q_blocks, stream);
}
