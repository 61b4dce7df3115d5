// Attention of a portion of a prompt over the paged cache, bfloat16, head sizes
// 64 and 128: a block takes 64 query tokens of one request and one query head and
// walks the keys 0 .. its last position in ascending tiles of 64 with an online
// softmax (queries are the tail of the keys they attend to, with an optional
// window).
//
// Five warps: warp 4 fetches key and value tiles by TMA (tensor map over the
// layer's pages seen as rows of d elements, 128-byte swizzle; the pages of a
// tile are looked up by its lanes in parallel) into a two-stage ring; warps 0..3
// each own 16 query rows and compute S = Q K^T and O += P V on mma.sync
// m16n8k16 (bfloat16 in, float32 accumulate) with fragments from ldmatrix.
// A row's arithmetic depends on its own position only: tile edges lie at
// multiples of 64 keys, and masked keys carry weight zero.
//
// Every wait is bounded; a wait that runs out records LS_DEV_WAIT_TIMEOUT.
#include <cuda.h>
#include <math_constants.h>

#include "common.cuh"

namespace {

constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr int BLOCK_M = 64;               // query tokens per block
constexpr int BLOCK_N = 64;               // keys per tile
constexpr int STAGES = 2;
constexpr int CONSUMERS = 4;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// HALVES = d / 64.  A stage holds K [HALVES][64 keys][128 B] then V the same.
template <int HALVES>
__global__ void __launch_bounds__((CONSUMERS + 1) * 32)
attention_prefill_mma_kernel(const __grid_constant__ CUtensorMap map, const __nv_bfloat16* __restrict__ q,
                             __nv_bfloat16* __restrict__ out, const int* __restrict__ work,
                             const int* __restrict__ block_table, int table_stride, int nq, int nkv,
                             int page_size, int num_pages, int window, float scale_log2, int* err) {
  ls_dependency_sync();
  constexpr int D = HALVES * 64;
  constexpr int KSTEPS = D / 16;
  constexpr int DTILES = D / 8;
  constexpr int NTILES = BLOCK_N / 8;
  constexpr int HALF_BYTES = BLOCK_N * 128;
  constexpr int KV_BYTES = HALVES * HALF_BYTES;          // K (or V) of one tile
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int Q_BYTES = BLOCK_M * D * 2;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + STAGES * STAGE_BYTES + Q_BYTES);
  uint64_t* full = bars;               // [STAGES] TMA bytes landed
  uint64_t* empty = bars + STAGES;     // [STAGES] all consumer warps are done with the stage

  // blocks are handed out head-fastest, so the tiles with the longest context (listed
  // first) start first for every head and the short ones fill the tail
  const int* w = work + (int64_t)blockIdx.y * 8;
  const int req_row = w[0], tok0 = w[1], ntok = w[2], pos0 = w[3];
  if (ntok == 0) return;
  const int h = blockIdx.x;
  const int kvh = h / (nq / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* table_row = block_table + (int64_t)req_row * table_stride;

  const int pos_last = pos0 + ntok - 1;
  const int key_lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;   // first key any row reads
  const int tile_first = key_lo / BLOCK_N;
  const int tile_end = pos_last / BLOCK_N + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CONSUMERS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the query tile, 16-byte chunks swizzled by the row
  if (warp < CONSUMERS) {
    for (int idx = threadIdx.x; idx < BLOCK_M * (D / 8); idx += CONSUMERS * 32) {
      const int row = idx / (D / 8), ch = idx % (D / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (row < ntok) v = *reinterpret_cast<const uint4*>(q + ((int64_t)(tok0 + row) * nq + h) * D + ch * 8);
      *reinterpret_cast<uint4*>(aligned + (q_smem - base) + row * (D * 2) + ((ch ^ (row & 7)) << 4)) = v;
    }
  }
  __syncthreads();

  if (warp == CONSUMERS) {
    // ---- producer ----
    const int rows_per_box = page_size < BLOCK_N ? page_size : BLOCK_N;
    const int boxes = BLOCK_N / rows_per_box;            // at most 8
    for (int tile = tile_first, it = 0; tile < tile_end; ++tile, ++it) {
      const int s = it % STAGES;
      const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
      const int c0 = tile * BLOCK_N;
      int page = 0;
      if (lane < boxes) {
        int key = c0 + lane * rows_per_box;
        if (key > pos_last) key = pos_last;              // past the last key: any page that exists
        if (key < key_lo) key = key_lo;                  // behind the window: pages may have been given back
        page = table_row[key / page_size];
        if (page < 0 || page >= num_pages) {
          ls_record_fault(err, LS_DEV_PAGE_RANGE, key);
          page = 0;
        }
      }
      if (!mbar_wait(&empty[s], phase ^ 1u)) {
        if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 600 + s);
        break;
      }
      const uint32_t stage = base + s * STAGE_BYTES;
      if (lane == 0) mbar_expect_tx(&full[s], STAGE_BYTES);
      for (int b = 0; b < boxes; ++b) {
        const int pg = __shfl_sync(0xffffffffu, page, b);
        if (lane == 0) {
          const int in_page = ((c0 + b * rows_per_box) % page_size) / rows_per_box * rows_per_box;
          const int y_k = ((pg * 2 + 0) * nkv + kvh) * page_size + in_page;
          const int y_v = ((pg * 2 + 1) * nkv + kvh) * page_size + in_page;
#pragma unroll
          for (int hh = 0; hh < HALVES; ++hh) {
            const uint32_t off = (uint32_t)(hh * HALF_BYTES + b * rows_per_box * 128);
            tma_load_2d(stage + off, &map, hh * 64, y_k, &full[s]);
            tma_load_2d(stage + KV_BYTES + off, &map, hh * 64, y_v, &full[s]);
          }
        }
      }
    }
    return;
  }

  // ---- consumers: warp owns query rows 16*warp .. +16; this thread rows r0 and r0 + 8 of them ----
  const int r0 = lane >> 2, cq = (lane & 3) * 2;
  const int row_a = warp * 16 + r0, row_b = row_a + 8;
  const int pos_a = pos0 + row_a, pos_b = pos0 + row_b;          // positions of this thread's rows
  const int lo_a = (window > 0 && pos_a - window + 1 > 0) ? pos_a - window + 1 : 0;
  const int lo_b = (window > 0 && pos_b - window + 1 > 0) ? pos_b - window + 1 : 0;
  const bool warp_live = warp * 16 < ntok;
  // last key any row of this warp reads, first key any of them reads
  const int warp_hi = pos0 + (warp * 16 + 15 < ntok ? warp * 16 + 15 : ntok - 1);
  const int warp_lo = (window > 0 && pos0 + warp * 16 - window + 1 > 0) ? pos0 + warp * 16 - window + 1 : 0;

  uint32_t qa[KSTEPS][4];
  {
    const int j = lane >> 3;
    const int row = warp * 16 + (j & 1) * 8 + (lane & 7);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int ch = ks * 2 + (j >> 1);
      ldmatrix_x4(q_smem + row * (D * 2) + ((ch ^ (row & 7)) << 4), qa[ks]);
    }
  }

  float acc[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};

  for (int tile = tile_first, it = 0; tile < tile_end; ++tile, ++it) {
    const int s = it % STAGES;
    const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
    const int c0 = tile * BLOCK_N;
    if (!mbar_wait(&full[s], phase)) {
      if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 700 + warp);
      break;
    }
    const uint32_t k_smem = base + s * STAGE_BYTES, v_smem = k_smem + KV_BYTES;
    // a tile that no row of this warp reads changes nothing: skip its arithmetic
    const bool tile_live = warp_live && c0 <= warp_hi && c0 + BLOCK_N > warp_lo;
    if (tile_live) {
      float sc[NTILES][4];
#pragma unroll
      for (int nt = 0; nt < NTILES; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const int half = ks / 4, chunk16 = (ks % 4) * 2, j = lane >> 3;
#pragma unroll
        for (int np = 0; np < NTILES / 2; ++np) {
          const int key = np * 16 + (j >> 1) * 8 + (lane & 7);
          const int ch = chunk16 + (j & 1);
          uint32_t b[4];
          ldmatrix_x4(k_smem + half * HALF_BYTES + key * 128 + ((ch ^ (key & 7)) << 4), b);
          mma_bf16(sc[np * 2 + 0], qa[ks], b[0], b[1]);
          mma_bf16(sc[np * 2 + 1], qa[ks], b[2], b[3]);
        }
      }
      // mask (only tiles that touch a row's edges need it), online softmax in base 2
      const bool need_mask = c0 + BLOCK_N - 1 > pos0 + warp * 16 || (window > 0 && c0 < warp_lo + 15 + 1);
      float tile_max[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int nt = 0; nt < NTILES; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = sc[nt][e] * scale_log2;
          if (need_mask) {
            const int key = c0 + nt * 8 + cq + (e & 1);
            const bool keep = (e < 2) ? (key <= pos_a && key >= lo_a && row_a < ntok)
                                      : (key <= pos_b && key >= lo_b && row_b < ntok);
            v = keep ? v : -CUDART_INF_F;
          }
          sc[nt][e] = v;
          tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
        }
      float alpha[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float m_new = fmaxf(m_run[r], tile_max[r]);
        alpha[r] = (m_run[r] == -CUDART_INF_F) ? (m_new == -CUDART_INF_F ? 1.f : 0.f) : exp2f(m_run[r] - m_new);
        m_run[r] = m_new;
      }
      float psum[2] = {0.f, 0.f};
      uint32_t pa[NTILES / 2][4];
#pragma unroll
      for (int nt = 0; nt < NTILES; ++nt) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[e] = (sc[nt][e] == -CUDART_INF_F) ? 0.f : exp2f(sc[nt][e] - m_run[e >> 1]);
          psum[e >> 1] += p[e];
        }
        pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
        psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
        l_run[r] = l_run[r] * alpha[r] + psum[r];
      }
#pragma unroll
      for (int i = 0; i < DTILES; ++i) {
        acc[i][0] *= alpha[0];
        acc[i][1] *= alpha[0];
        acc[i][2] *= alpha[1];
        acc[i][3] *= alpha[1];
      }
      // values of keys past the block's last position are whatever the page holds; their
      // weight is 0, but 0 * inf is not.  Each warp clears those rows of V itself before
      // it multiplies (the warps write the same zeros, so they need no order among them).
      if (c0 + BLOCK_N > pos_last + 1) {
        const int valid = pos_last + 1 - c0;
        for (int idx = lane; idx < HALVES * BLOCK_N * 8; idx += 32) {
          const int half = idx / (BLOCK_N * 8), key = (idx / 8) % BLOCK_N, ch = idx & 7;
          if (key >= valid)
            *reinterpret_cast<uint4*>(aligned + (v_smem - base) + half * HALF_BYTES + key * 128 + ch * 16) =
                make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }
#pragma unroll
      for (int kstep = 0; kstep < BLOCK_N / 16; ++kstep) {
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
          const int j = lane >> 3;
          const int key = kstep * 16 + (j & 1) * 8 + (lane & 7);
          const int dim8 = dp * 2 + (j >> 1);
          const int half = dim8 / 8, ch = dim8 % 8;
          uint32_t b[4];
          ldmatrix_x4_trans(v_smem + half * HALF_BYTES + key * 128 + ((ch ^ (key & 7)) << 4), b);
          mma_bf16(acc[dp * 2 + 0], pa[kstep], b[0], b[1]);
          mma_bf16(acc[dp * 2 + 1], pa[kstep], b[2], b[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }

  // write O = acc / l for the rows that exist
  const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
  const float inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  if (row_a < ntok) {
    __nv_bfloat16* o = out + ((int64_t)(tok0 + row_a) * nq + h) * D;
#pragma unroll
    for (int i = 0; i < DTILES; ++i)
      *reinterpret_cast<uint32_t*>(o + i * 8 + cq) = pack_bf16(acc[i][0] * inv_a, acc[i][1] * inv_a);
  }
  if (row_b < ntok) {
    __nv_bfloat16* o = out + ((int64_t)(tok0 + row_b) * nq + h) * D;
#pragma unroll
    for (int i = 0; i < DTILES; ++i)
      *reinterpret_cast<uint32_t*>(o + i * 8 + cq) = pack_bf16(acc[i][2] * inv_b, acc[i][3] * inv_b);
  }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
  }
  return fn;
}

template <int HALVES>
int launch(const CUtensorMap& map, const void* q, void* out, const int* work, int n_work,
           const int* block_table, int table_stride, int nq, int nkv, int page_size, int num_pages,
           int window, float scale, int* err, cudaStream_t stream) {
  const size_t smem = (size_t)STAGES * 2 * HALVES * BLOCK_N * 128 + (size_t)BLOCK_M * HALVES * 128 + 64 + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_mma_kernel<HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return LS_E_SMEM;
    configured = true;
  }
  dim3 grid(nq, n_work);
  ls_launch(attention_prefill_mma_kernel<HALVES>, grid, (CONSUMERS + 1) * 32, smem, stream, 
      map, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, work, block_table, table_stride, nq, nkv,
      page_size, num_pages, window, scale * 1.4426950408889634f, err);
  return ls_launch_status();
}

}  // namespace

LS_API int ls_attention_prefill_tile_tokens() { return BLOCK_M; }

// bfloat16 only; d 64 or 128; page sizes 8, 16, 32, 64.  work items as for
// ls_attention_tile, with up to 64 tokens each (splits and slots are not used).
// Returns LS_E_SIZE for anything else, having launched nothing.
LS_API int ls_attention_prefill_mma(const void* q, const void* pages, void* out, const int* work,
                                    int n_work, const int* block_table, int table_stride, int nq,
                                    int nkv, int d, int page_size, int num_pages, int window,
                                    float scale, int* err, cudaStream_t stream) {
  if (n_work <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv || n_work > 65535) return LS_E_SIZE;
  if (d != 64 && d != 128) return LS_E_SIZE;
  if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return LS_E_SIZE;
  const int64_t rows = (int64_t)num_pages * 2 * nkv * page_size;
  if (rows > 2147483647LL || ((uintptr_t)pages & 127)) return LS_E_SIZE;
  EncodeTiled enc = encode_fn();
  if (enc == nullptr) return LS_E_SIZE;
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)d * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)(page_size < BLOCK_N ? page_size : BLOCK_N)};
  cuuint32_t elem[2] = {1, 1};
  if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return LS_E_SIZE;
  if (d == 64)
    return launch<1>(map, q, out, work, n_work, block_table, table_stride, nq, nkv, page_size, num_pages,
                     window, scale, err, stream);
  return launch<2>(map, q, out, work, n_work, block_table, table_stride, nq, nkv, page_size, num_pages,
                   window, scale, err, stream);
}
