// Decode attention over the paged cache for bfloat16, head sizes 64 and 128:
// one query token, one 256-key split, one kv head with its whole group of
// query heads (up to 16, padded to the 16 rows of an MMA tile).
//
// A block has four warps that work alone until the end: warp w takes the keys
// [32*(4*i + w), +32) of the split for i = 0, 1.  Its lane 0 fetches the pages
// of those keys by TMA (tensor map over the layer's pages seen as rows of d
// elements, 128-byte swizzle) into the warp's own shared memory, K and V on
// barriers of their own so that V arrives while QK^T is computed.  Scores and
// the PV product run on mma.sync m16n8k16 (bfloat16 in, float32 accumulate),
// fragments read with ldmatrix.  The four warps' partial results are folded in
// warp order, and the split's (acc, m, l) goes to the scratch that
// ls_attention_combine folds in ascending split order.
//
// Every wait is bounded: a wait that runs out records LS_DEV_WAIT_TIMEOUT and
// the warp goes on with whatever shared memory holds (finite garbage, masked
// where possible); the host raises after the step.
#include <cuda.h>
#include <math_constants.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int CHUNK = 32;                 // keys a warp handles per iteration
constexpr int WARPS = 4;

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

// HALVES = d / 64.  Shared memory of a warp: K [HALVES][32 keys][128 B], then V the same.
template <int HALVES>
__global__ void __launch_bounds__(WARPS * 32, 3)
attention_decode_mma_kernel(const __grid_constant__ CUtensorMap map, const __nv_bfloat16* __restrict__ q,
                            float* __restrict__ part_acc, float* __restrict__ part_ml,
                            const int* __restrict__ work, const int* __restrict__ block_table,
                            int table_stride, int nq, int nkv, int page_size, int num_pages, int window,
                            float scale, int* err) {
  // The work list, the block table and every key older than this step's token are there
  // before the step's first kernel starts, so the first chunks are fetched while the kernel
  // before this one (which writes the token's own key and value, and q) still runs.
  ls_dependency_trigger();
  constexpr int D = HALVES * 64;
  constexpr int KSTEPS = D / 16;                 // k-steps of QK^T
  constexpr int DTILES = D / 8;                  // n-tiles of PV
  constexpr int HALF_BYTES = CHUNK * 128;        // one half of K (or V) of a chunk
  constexpr int WARP_BYTES = 2 * HALVES * HALF_BYTES;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + WARPS * WARP_BYTES);   // [WARPS][2]
  const uint32_t q_smem = base + WARPS * WARP_BYTES + 128;                      // [16 rows][D] bfloat16

  const int* w = work + (int64_t)blockIdx.x * 8;
  const int ntok = w[2];
  if (ntok == 0) return;                         // padding item of a captured launch
  const int req_row = w[0], tok = w[1], pos = w[3], split = w[4], slot = w[6];
  const int kvh = blockIdx.y;
  const int group = nq / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* table_row = block_table + (int64_t)req_row * table_stride;
  const int row_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int s_lo = split * LS_SPLIT;
  int s_hi = s_lo + LS_SPLIT;
  if (s_hi > pos + 1) s_hi = pos + 1;

  const uint32_t k_smem = base + warp * WARP_BYTES;
  const uint32_t v_smem = k_smem + HALVES * HALF_BYTES;
  uint64_t* bar_k = bars + warp * 2;
  uint64_t* bar_v = bar_k + 1;
  if (lane == 0) {
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  const int r0 = lane >> 2, cq = (lane & 3) * 2;   // this thread holds rows r0 and r0 + 8

  float acc[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};

  const int rows_per_box = page_size < CHUNK ? page_size : CHUNK;
  const int boxes = CHUNK / rows_per_box;
  uint32_t parity = 0;

  // the pages of this warp's chunks, looked up once: lane 4 * i + b holds box b of chunk i
  const int n_iter = LS_SPLIT / (WARPS * CHUNK);
  int my_page = 0;
  {
    const int i = lane >> 2, b = lane & 3;
    if (i < n_iter && b < boxes) {
      const int c0 = s_lo + (i * WARPS + warp) * CHUNK;
      if (c0 < s_hi && c0 + CHUNK > row_lo) {
        int key = c0 + b * rows_per_box;
        if (key >= s_hi) key = s_hi - 1;          // beyond the split's end: any page that exists
        if (key < row_lo) key = row_lo;           // behind the window: pages may have been given back
        my_page = table_row[key / page_size];
        if (my_page < 0 || my_page >= num_pages) {
          ls_record_fault(err, LS_DEV_PAGE_RANGE, key);
          my_page = 0;
        }
      }
    }
  }

  // issue the loads of chunk i (first key c0): K on bar_k, V on bar_v.  Called by the whole warp.
  // Every box is issued by a lane of its own: a thread gets one TMA instruction out about
  // every 300 ns, whatever the box's size, so one lane issuing a chunk's up to 16 boxes would
  // spend several microseconds on it.
  auto issue = [&](int i, int c0, bool want_k, bool want_v) {
    const uint32_t bytes = (uint32_t)(HALVES * HALF_BYTES);
    if (lane == 0) {
      if (want_k) mbar_expect_tx(bar_k, bytes);
      if (want_v) mbar_expect_tx(bar_v, bytes);
    }
    __syncwarp();
    const int b = lane / (2 * HALVES), h = (lane >> 1) % HALVES, is_v = lane & 1;    // this lane's box
    const int page = __shfl_sync(0xffffffffu, my_page, i * 4 + (b < boxes ? b : 0));
    if (b < boxes && (is_v ? want_v : want_k)) {
      const int in_page = ((c0 + b * rows_per_box) % page_size) / rows_per_box * rows_per_box;
      const int y = ((page * 2 + is_v) * nkv + kvh) * page_size + in_page;
      const uint32_t off = (uint32_t)(h * HALF_BYTES + b * rows_per_box * 128);
      tma_load_2d((is_v ? v_smem : k_smem) + off, &map, h * 64, y, is_v ? bar_v : bar_k);
    }
  };

  // chunks of this warp: keys c0 = s_lo + (i * WARPS + warp) * CHUNK that are not wholly outside [row_lo, s_hi)
  auto chunk_start = [&](int i) { return s_lo + (i * WARPS + warp) * CHUNK; };
  auto chunk_live = [&](int i) {
    const int c0 = chunk_start(i);
    return i < n_iter && c0 < s_hi && c0 + CHUNK > row_lo;
  };

  int it = 0;
  while (it < n_iter && !chunk_live(it)) ++it;
  // a chunk that holds the step's own token waits for the kernel that writes it
  const bool first_early = it < n_iter && chunk_start(it) + CHUNK <= pos;
  if (first_early) issue(it, chunk_start(it), true, true);
  ls_dependency_wait();
  if (it < n_iter && !first_early) issue(it, chunk_start(it), true, true);

  // rows of the MMA tile are the group's query heads (zero rows pad it to 16); the
  // tile sits in shared memory with its 16-byte chunks swizzled by the row
  {
    const __nv_bfloat16* qb = q + ((int64_t)tok * nq + kvh * group) * D;
    for (int idx = threadIdx.x; idx < 16 * (D / 8); idx += WARPS * 32) {
      const int row = idx / (D / 8), ch = idx % (D / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (row < group) v = *reinterpret_cast<const uint4*>(qb + row * D + ch * 8);
      *reinterpret_cast<uint4*>(aligned + (q_smem - base) + row * (D * 2) + ((ch ^ (row & 7)) << 4)) = v;
    }
  }
  __syncthreads();

  while (it < n_iter) {
    const int c0 = chunk_start(it);
    int next = it + 1;
    while (next < n_iter && !chunk_live(next)) ++next;

    if (!mbar_wait(bar_k, parity)) {
      if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 400 + warp);
    }
    // scores: 16 rows x 32 keys
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int half = ks / 4;
      const int chunk16 = (ks % 4) * 2;          // 16-byte chunk of the 128-byte row
      const int j = lane >> 3;                   // matrix this lane addresses
      uint32_t qa[4];
      {
        const int row = (j & 1) * 8 + (lane & 7);
        const int ch = ks * 2 + (j >> 1);
        ldmatrix_x4(q_smem + row * (D * 2) + ((ch ^ (row & 7)) << 4), qa);
      }
#pragma unroll
      for (int np = 0; np < 2; ++np) {           // two key tiles per ldmatrix.x4
        const int key = np * 16 + (j >> 1) * 8 + (lane & 7);
        const int ch = chunk16 + (j & 1);
        const uint32_t addr = k_smem + half * HALF_BYTES + key * 128 + ((ch ^ (key & 7)) << 4);
        uint32_t b[4];
        ldmatrix_x4(addr, b);
        mma_bf16(s[np * 2 + 0], qa, b[0], b[1]);
        mma_bf16(s[np * 2 + 1], qa, b[2], b[3]);
      }
    }
    __syncwarp();
    // K is consumed: fetch the next chunk's K while the softmax and PV of this one run
    const bool more = next < n_iter;
    if (more) {
      // the generic-proxy reads above are ordered before the async-proxy writes (every lane issues)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue(next, chunk_start(next), true, false);
    }

    // mask, online softmax (rows r0 and r0 + 8; columns nt * 8 + cq, +1)
    float tile_max[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = c0 + nt * 8 + cq + (e & 1);
        const bool keep = key < s_hi && key >= row_lo;
        s[nt][e] = keep ? s[nt][e] * scale : -CUDART_INF_F;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], s[nt][e]);
      }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float m_new = fmaxf(m_run[r], tile_max[r]);
      alpha[r] = (m_run[r] == -CUDART_INF_F) ? (m_new == -CUDART_INF_F ? 1.f : 0.f) : expf(m_run[r] - m_new);
      m_run[r] = m_new;
    }
    float psum[2] = {0.f, 0.f};
    uint32_t pa[2][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float m = m_run[e >> 1];
        p[e] = (s[nt][e] == -CUDART_INF_F) ? 0.f : expf(s[nt][e] - m);
        psum[e >> 1] += p[e];
      }
      // C fragments of two adjacent key tiles form the A fragment of one 16-key step
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

    if (!mbar_wait(bar_v, parity)) {
      if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 500 + warp);
    }
    // Values of masked keys (past the row's last key, behind its window) are whatever
    // the page holds; their weight is 0, but 0 * inf is not: clear those rows.
    {
      const int valid_hi = s_hi - c0, valid_lo = row_lo - c0;
      if (valid_hi < CHUNK || valid_lo > 0) {
        for (int idx = lane; idx < HALVES * CHUNK * 8; idx += 32) {
          const int half = idx / (CHUNK * 8), key = (idx / 8) % CHUNK, ch = idx & 7;
          if (key >= valid_hi || key < valid_lo)
            *reinterpret_cast<uint4*>(aligned + (v_smem - base) + half * HALF_BYTES + key * 128 + ch * 16) =
                make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }
    }
#pragma unroll
    for (int kstep = 0; kstep < 2; ++kstep) {    // 16 keys each
#pragma unroll
      for (int dp = 0; dp < DTILES / 2; ++dp) {  // two 8-dim tiles per ldmatrix.x4.trans
        const int j = lane >> 3;
        const int key = kstep * 16 + (j & 1) * 8 + (lane & 7);
        const int dim8 = dp * 2 + (j >> 1);      // 8-dim tile index
        const int half = dim8 / 8, ch = dim8 % 8;
        const uint32_t addr = v_smem + half * HALF_BYTES + key * 128 + ((ch ^ (key & 7)) << 4);
        uint32_t b[4];
        ldmatrix_x4_trans(addr, b);
        mma_bf16(acc[dp * 2 + 0], pa[kstep], b[0], b[1]);
        mma_bf16(acc[dp * 2 + 1], pa[kstep], b[2], b[3]);
      }
    }
    __syncwarp();
    if (more) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue(next, chunk_start(next), false, true);
    }
    parity ^= 1u;
    it = next;
  }

  // fold the four warps in warp order; rows below `group` only
  __syncthreads();
  float* red = reinterpret_cast<float*>(aligned);      // [WARPS][group][D + 2], reuses the K/V space
  const int stride = D + 2;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r0 + r * 8;
    if (row < group) {
      float* dst = red + ((size_t)warp * group + row) * stride;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) {
        dst[i * 8 + cq] = acc[i][r * 2];
        dst[i * 8 + cq + 1] = acc[i][r * 2 + 1];
      }
      if ((lane & 3) == 0) {
        dst[D] = m_run[r];
        dst[D + 1] = l_run[r];
      }
    }
  }
  __syncthreads();
  for (int u = threadIdx.x; u < group * D; u += WARPS * 32) {
    const int g = u / D, c = u - g * D;
    float m = -CUDART_INF_F, l = 0.f, a = 0.f;
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) {
      const float* src = red + ((size_t)wi * group + g) * stride;
      const float m_w = src[D];
      if (m_w == -CUDART_INF_F) continue;
      const float m_new = fmaxf(m, m_w);
      const float sa = (m == -CUDART_INF_F) ? 0.f : expf(m - m_new);
      const float sb = expf(m_w - m_new);
      a = a * sa + src[c] * sb;
      l = l * sa + src[D + 1] * sb;
      m = m_new;
    }
    const int64_t o = ((int64_t)slot * nq + kvh * group + g);
    part_acc[o * D + c] = a;
    if (c == 0) {
      part_ml[o * 2 + 0] = m;
      part_ml[o * 2 + 1] = l;
    }
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
int launch(const CUtensorMap& map, const void* q, float* part_acc, float* part_ml, const int* work,
           int n_work, const int* block_table, int table_stride, int nq, int nkv, int page_size,
           int num_pages, int window, float scale, int* err, cudaStream_t stream) {
  const size_t smem = (size_t)WARPS * 2 * HALVES * CHUNK * 128 + 128 + 16 * HALVES * 128 + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_decode_mma_kernel<HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return LS_E_SMEM;
    configured = true;
  }
  dim3 grid(n_work, nkv);
  LS_COUNT(LS_K_ATTENTION_DECODE_MMA), ls_launch(attention_decode_mma_kernel<HALVES>, grid, WARPS * 32, smem, stream, 
      map, (const __nv_bfloat16*)q, part_acc, part_ml, work, block_table, table_stride, nq, nkv, page_size,
      num_pages, window, scale, err);
  return ls_launch_status();
}

}  // namespace

// bfloat16 only; d 64 or 128; group (nq / nkv) up to 16; page sizes 8, 16, 32, 64.
// Returns LS_E_SIZE for anything else, having launched nothing.
LS_API int ls_attention_decode_mma(const void* q, const void* pages, float* part_acc, float* part_ml,
                                   const int* work, int n_work, const int* block_table,
                                   int table_stride, int nq, int nkv, int d, int page_size,
                                   int num_pages, int window, float scale, int* err,
                                   cudaStream_t stream) {
  if (n_work <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv || nq / nkv > 16 || nkv > 65535) return LS_E_SIZE;
  if (d != 64 && d != 128) return LS_E_SIZE;
  if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return LS_E_SIZE;
  const int64_t rows = (int64_t)num_pages * 2 * nkv * page_size;
  if (rows > 2147483647LL || ((uintptr_t)pages & 127)) return LS_E_SIZE;
  EncodeTiled enc = encode_fn();
  if (enc == nullptr) return LS_E_SIZE;
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)d * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)(page_size < CHUNK ? page_size : CHUNK)};
  cuuint32_t elem[2] = {1, 1};
  if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return LS_E_SIZE;
  if (d == 64)
    return launch<1>(map, q, part_acc, part_ml, work, n_work, block_table, table_stride, nq, nkv, page_size,
                     num_pages, window, scale, err, stream);
  return launch<2>(map, q, part_acc, part_ml, work, n_work, block_table, table_stride, nq, nkv, page_size,
                   num_pages, window, scale, err, stream);
}

LS_API const char* ls_constants_attention_decode_mma() {
  static char buf[256];
  static const LsConstant c[] = {{"attention_decode_mma.split_keys", LS_SPLIT}, {"attention_decode_mma.warp_keys", CHUNK},
                                 {"attention_decode_mma.warps", WARPS}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}
