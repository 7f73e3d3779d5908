// bfloat16 prompt attention with sigmoid weights inside chunks, on the tensor cores.
//
//   s_ij = (q_i . k_j) * scale + bias[head]
//   j visible to i  iff  j <= i and floor(i / chunk) == floor(j / chunk)   (chunk 0: j <= i)
//   o_i = out_scale * sigmoid(gate_i[head]) * sum_j sigmoid(s_ij) v_j      (no gate: 1)
//
// A 64-row block of one sequence's queries for one head walks the cache pages from the one
// that holds the start of its first query's chunk to the one of its last query, 64 keys at a
// time, two pages in flight; the four warps own 16 query rows each; mma.sync.m16n8k16 with
// 32-bit accumulation. Scores and weights are 32-bit; a weight is rounded to bfloat16 only as
// the operand of the product with the values. There is no running maximum and no sum to
// divide by, so a page's share is simply added. A block that straddles a chunk's edge masks
// by row: the first key a row sees is the start of that row's own chunk. Key rows beyond the
// sequence's length are read as zeros.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace {

using namespace fb_mma;

struct SigmoidParams {
  const __nv_bfloat16* q; long long q_stride;   // head h at h * DK
  __nv_bfloat16* out; long long out_stride;     // head h at h * DV
  const int* cu_tokens;  // [n_seqs + 1]
  const int* kv_lens;    // [n_seqs]: length after this step
  const int* page_table; int max_pages;
  const __nv_bfloat16* k; const __nv_bfloat16* v;
  long long k_page, k_head, v_page, v_head;
  const float* head_bias;              // [H] or null
  const float* gate; long long gate_ld;  // raw gate values [T, >= H] or null
  int n_seqs, H, G, chunk;
  float scale, out_scale;
};

template <int DK, int DV>
__global__ void __launch_bounds__(THREADS) attn_sigmoid_mma_kernel(const SigmoidParams p) {
  fb_pdl_wait();
  constexpr int PK = pitch_of(DK), PV = pitch_of(DV);
  constexpr int KT = DK / 16;  // k-steps of Q.K^T
  constexpr int NT = DV / 8;   // n-tiles of P.V
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
  const int chunk = p.chunk;
  const int first_key = chunk > 0 ? (pos0 / chunk) * chunk : 0;
  const int pg_first = first_key / FB_PAGE, pg_end = last_key / FB_PAGE + 1;
  const int* pages = p.page_table + (size_t)seq * p.max_pages;

  auto load_kv = [&](int stage, int pg) {
    const long long page = pages[pg];
    const int valid = min(FB_PAGE, kv_len - pg * FB_PAGE);
    load_cols<PK>(sK + stage * 64 * PK, p.k + page * p.k_page + kvh * p.k_head, DK, 64, valid, DK, 0);
    load_cols<PV>(sV + stage * 64 * PV, p.v + page * p.v_page + kvh * p.v_head, DV, 64, valid, DV, 0);
  };

  load_cols<PK>(sQ, p.q + (long long)(tok0 + row0) * p.q_stride + (long long)head * DK, p.q_stride,
                64, rows_valid, DK, 0);
  load_kv(0, pg_first);
  cp_async_commit();

  uint32_t qf[KT][4];
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  // rows g and g + 8 of the warp's 16: their positions and the first keys they see
  int qpos[2], qlo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    qpos[r] = pos0 + warp * 16 + g + r * 8;
    qlo[r] = chunk > 0 ? (qpos[r] / chunk) * chunk : 0;
  }
  const int w_first = pos0 + warp * 16, w_last = w_first + 15;
  const int w_lo_first = chunk > 0 ? (w_first / chunk) * chunk : 0;  // first key any row sees
  const int w_lo_last = chunk > 0 ? (w_last / chunk) * chunk : 0;    // first key every row sees
  const float bias2 = (p.head_bias != nullptr ? p.head_bias[head] : 0.f) * LOG2E;
  const float scale2 = p.scale * LOG2E;

  for (int pg = pg_first; pg < pg_end; ++pg) {
    const int st = (pg - pg_first) & 1;
    if (pg + 1 < pg_end) load_kv(st ^ 1, pg + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (pg == pg_first) {
#pragma unroll
      for (int k = 0; k < KT; ++k)
        ldsm_x4(qf[k], smem_u32(sQ + Swz<PK>::off(warp * 16 + (lane & 15), k * 16 + (lane >> 4) * 8)));
    }
    const int key0 = pg * FB_PAGE;
    if (key0 <= w_last && key0 + FB_PAGE - 1 >= w_lo_first) {  // else no row of the warp sees these keys
      const __nv_bfloat16* tK = sK + st * 64 * PK;
      const __nv_bfloat16* tV = sV + st * 64 * PV;
      const bool need_mask = key0 + FB_PAGE - 1 > w_first || key0 < w_lo_last;
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int k = 0; k < KT; ++k) {
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {  // two n-tiles (16 keys) per ldmatrix.x4
          uint32_t b[4];
          ldsm_x4(b, smem_u32(tK + Swz<PK>::off(n2 * 16 + (lane & 7) + (lane >> 4) * 8,
                                                k * 16 + ((lane >> 3) & 1) * 8)));
          mma_bf16(s[2 * n2], qf[k], b[0], b[1]);
          mma_bf16(s[2 * n2 + 1], qf[k], b[2], b[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // sigmoid(x) = 1 / (1 + 2^(-x log2 e)); beyond 2^126 the weight is below the
          // smallest normal number
          const float ex = exp2f(fminf(-fmaf(s[n][e], scale2, bias2), 126.0f));
          float w = __fdividef(1.0f, 1.0f + ex);
          if (need_mask) {
            const int key = key0 + n * 8 + 2 * t + (e & 1);
            if (key > qpos[e >> 1] || key < qlo[e >> 1]) w = 0.f;
          }
          s[n][e] = w;
        }
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int n2 = 0; n2 < NT / 2; ++n2) {
          uint32_t b[4];
          ldsm_x4_trans(b, smem_u32(tV + Swz<PV>::off(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                     n2 * 16 + (lane >> 4) * 8)));
          mma_bf16(o[2 * n2], pa, b[0], b[1]);
          mma_bf16(o[2 * n2 + 1], pa, b[2], b[3]);
        }
      }
    }
    __syncthreads();  // the stage is refilled two iterations on
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + r * 8;
    if (row >= rows_valid) continue;
    const long long tok = tok0 + row0 + row;
    float mul = p.out_scale;
    if (p.gate != nullptr) mul *= 1.0f / (1.0f + expf(-__ldcg(p.gate + tok * p.gate_ld + head)));
    __nv_bfloat16* dst = p.out + tok * p.out_stride + (long long)head * DV;
#pragma unroll
    for (int n = 0; n < NT; ++n)
      *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) =
          pack_bf16(o[n][2 * r] * mul, o[n][2 * r + 1] * mul);
  }
}

template <int DK, int DV>
int launch_sigmoid(const SigmoidParams& p, int q_blocks, cudaStream_t stream) {
  constexpr int PK = pitch_of(DK), PV = pitch_of(DV);
  const size_t smem = (size_t)(3 * 64 * PK + 2 * 64 * PV) * sizeof(__nv_bfloat16);
  static bool seen[64];
  if (smem > 48 * 1024 && fb_first_use_on_device(seen))
    cudaFuncSetAttribute(attn_sigmoid_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
  fb_launch(attn_sigmoid_mma_kernel<DK, DV>, dim3(q_blocks, p.H), dim3(THREADS), smem, stream, p);
  return fb_check_launch("attention_sigmoid_mma");
}
}  // namespace

// Whether a (key size, value size) combination has a kernel here.
FB_API int fb_attention_sigmoid_mma_fits(int DK, int DV) {
  return (DK == 32 || DK == 64 || DK == 96 || DK == 128) && (DV == 32 || DV == 64 || DV == 128) &&
         (DK == DV || (DK == 64 && DV == 128) || (DK == 128 && DV == 64) || (DK == 96 && DV == 64) ||
          (DK == 32 && (DV == 64 || DV == 128)));
}

FB_API int fb_attention_sigmoid_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                    const int* cu_tokens, const int* kv_lens, const int* page_table,
                                    int max_pages, const void* k_cache, const void* v_cache,
                                    long long k_page, long long k_head, long long v_page,
                                    long long v_head, const float* head_bias, const float* gate,
                                    long long gate_ld, float scale, float out_scale, int chunk,
                                    int n_seqs, int q_blocks, int H, int G, int DK, int DV,
                                    cudaStream_t stream) {
  FB_REQUIRE(n_seqs >= 0 && q_blocks >= 0 && H > 0 && G > 0 && H % G == 0 && chunk >= 0 && H <= 65535,
             "attention_sigmoid_mma: bad sizes");
  FB_REQUIRE(fb_attention_sigmoid_mma_fits(DK, DV),
             "attention_sigmoid_mma: no kernel for keys of %d and values of %d", DK, DV);
  FB_REQUIRE(page_table != nullptr && max_pages > 0, "attention_sigmoid_mma: no page table");
  FB_REQUIRE(((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 == 0 &&
             q_stride % 8 == 0 && out_stride % 2 == 0 && k_page % 8 == 0 && k_head % 8 == 0 &&
             v_page % 8 == 0 && v_head % 8 == 0,
             "attention_sigmoid_mma: rows must start on 16-byte boundaries");
  if (n_seqs == 0 || q_blocks == 0) return 0;
  SigmoidParams p{(const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, cu_tokens,
                  kv_lens, page_table, max_pages, (const __nv_bfloat16*)k_cache,
                  (const __nv_bfloat16*)v_cache, k_page, k_head, v_page, v_head, head_bias, gate,
                  gate_ld, n_seqs, H, G, chunk, scale, out_scale};
#define FB_SIG(DK_, DV_) \
  if (DK == DK_ && DV == DV_) return launch_sigmoid<DK_, DV_>(p, q_blocks, stream)
  FB_SIG(32, 32); FB_SIG(64, 64); FB_SIG(128, 128); FB_SIG(64, 128); FB_SIG(128, 64);
  FB_SIG(96, 64); FB_SIG(32, 64); FB_SIG(32, 128);
#undef FB_SIG
  return fb_fail(1, "attention_sigmoid_mma: no kernel");
}
