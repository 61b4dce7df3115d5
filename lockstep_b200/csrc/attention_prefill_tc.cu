// Attention of a portion of a prompt over the paged cache on the 5th-generation
// tensor cores: bfloat16, head sizes 64 and 128.  A block takes 128 query tokens of
// one request and one query head (a token is a row of the MMA tile, a lane of
// tensor memory, and a thread of the softmax warps) and walks the keys in
// ascending tiles of 128, whose edges lie at multiples of 128 keys whatever the
// portion, so a row's arithmetic depends on its own position only.
//
//   S = Q K^T     tcgen05.mma, Q [128 x d] and the key tile [128 x d] K-major in
//                 shared memory (TMA, 128-byte swizzle), S in tensor memory
//   softmax       the threads of a row read it from S with tcgen05.ld: maximum,
//                 p = exp2(s * scale * log2 e - m_ref), the running sum l in registers; P
//                 rounded to bfloat16 goes back to tensor memory (tcgen05.st), two keys a column
//   PV            tcgen05.mma with P [128 x 128] as the A operand in tensor memory and the
//                 value tile [128 keys x d] as it lies in the cache (MN-major) in shared
//                 memory, adding to O in tensor memory over all tiles.  m_ref follows the
//                 row's maximum lazily (when it has grown by more than 8, a factor 256, the
//                 row of O is scaled and m_ref moved); O / l does not depend on m_ref.
//
// Nineteen warps: warp 0 fetches Q once and the key tiles, warp 18 the value tiles, into
// two stages each (a lane per page of a tile: look-up and TMA box), warp 1 issues the MMAs
// (S of the next tile before PV of this one, so the tensor cores work while the
// softmax runs; S and P have two buffers each in tensor memory), warps 2..17 are the
// softmax, four threads per row: each has 32 keys of a tile and a quarter of the head's
// dimensions; they share the row's maximum through shared memory.  (With two threads per
// row the softmax warps, two to a scheduler, were short of issue slots.)  Every wait is bounded; a wait that runs out records
// LS_DEV_WAIT_TIMEOUT and the block winds down and frees its tensor memory.
#include <cuda.h>
#include <math_constants.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int BLOCK_M = 128;              // query tokens per block
constexpr int BLOCK_N = 128;              // keys per tile
constexpr int STAGES = 2;
constexpr int UMMA_K = 16;
constexpr int HALF_BYTES = 128 * 128;     // 128 rows of 64 elements
constexpr uint32_t TMEM_COLS = 512;
constexpr int GROUPS = 4;                 // softmax threads per row (warpgroups of the softmax)
constexpr int THREADS = (3 + 4 * GROUPS) * 32;
constexpr int V_WARP = 2 + 4 * GROUPS;    // the warp that fetches the value tiles

// MN-major operand (the value tile as it lies in the cache: a key is a row of 128 bytes = 64
// elements of d): blocks of 64 elements of d are `block_stride` bytes apart (leading offset),
// groups of 8 keys 1024 bytes (stride offset); 128-byte swizzle
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t saddr, uint32_t block_stride) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((block_stride >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// the same with the A operand in tensor memory (row = lane, two bfloat16 of neighbouring k a column)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
        "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(taddr)
      : "memory");
}
// N columns (a multiple of 16) of this thread's lane to or from registers
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r) {
  static_assert(N % 16 == 0, "columns in sixteens");
#pragma unroll
  for (int c = 0; c + 32 <= N; c += 32) tmem_ld32(taddr + c, r + c);
  if constexpr (N % 32) tmem_ld16(taddr + N - 16, r + N - 16);
}
template <int N>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t* r) {
  static_assert(N % 16 == 0, "columns in sixteens");
#pragma unroll
  for (int c = 0; c + 32 <= N; c += 32) tmem_st32(taddr + c, r + c);
  if constexpr (N % 32) tmem_st16(taddr + N - 16, r + N - 16);
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 2^x on the special-function unit, one instruction (inputs here are <= 0 or -inf)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two float32 lanes an instruction (sm_100: fma / add on pairs of registers) and the maximum of
// three: the softmax warps are short of issue slots, and each of these halves an instruction
// count without changing a result (every lane is rounded as the single instruction rounds it).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (x, y) = (a x + c, a y + c)
__device__ __forceinline__ void fma2(float& x, float& y, float a, float c) {
  uint64_t xy, aa, cc, r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(xy) : "f"(x), "f"(y));
  asm("mov.b64 %0, {%1, %1};" : "=l"(aa) : "f"(a));
  asm("mov.b64 %0, {%1, %1};" : "=l"(cc) : "f"(c));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(xy), "l"(aa), "l"(cc));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(r));
}
// (x, y) += (a, b)
__device__ __forceinline__ void add2(float& x, float& y, float a, float b) {
  uint64_t xy, ab, r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(xy) : "f"(x), "f"(y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(ab) : "f"(a), "f"(b));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(xy), "l"(ab));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(r));
}

// One work item of a block: up to 128 tokens of a request (rows of the MMA tile) and one query head.
struct Item {
  const int* table_row;
  int tok0, ntok, pos0, h, kvh;
  int pos_last, key_lo, tile_first, n_tiles;
};

// HALVES = d / 64.  Shared memory: Q [HALVES][128 rows][128 B]; two stages of K and of V
// [HALVES][128 keys][128 B]; barriers.  Tensor memory: two S buffers, O, two P buffers (bfloat16).
//
// The kernel is persistent: a block per SM walks the items (work item x head, longest context
// first) in rounds, round r handing item r * blocks + b to block b, and every other round in the
// reverse order, so that a block with a long item gets a short one next.  Barriers, stages and
// buffers count on over the items of a block (tile counter `gt`), the producers run ahead into
// the next item's Q and first tiles while the softmax of the last tile still runs, and the
// tensor memory is allocated once: an item after the first does not pay a block's start again.
template <int HALVES>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            __nv_bfloat16* __restrict__ out, const int* __restrict__ work, int n_work,
                            const int* __restrict__ block_table, int table_stride, int nq, int nkv, int page_size,
                            int num_pages, int window, float scale_log2, int* err) {
  ls_dependency_trigger();
  constexpr int D = HALVES * 64;
  constexpr int KV_BYTES = HALVES * HALF_BYTES;          // K (or V) of one tile; also Q
  // tensor memory: two S buffers, O, and two P buffers (bfloat16, two keys a column)
  constexpr uint32_t S_COL = 0, O_COL = 2 * BLOCK_N, P_COL = O_COL + 128, P_COLS = BLOCK_N / 2;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;
  const uint32_t k_smem = q_smem + KV_BYTES;             // [STAGES]
  const uint32_t v_smem = k_smem + STAGES * KV_BYTES;    // [STAGES]
  const uint32_t bars_smem = v_smem + STAGES * KV_BYTES;
  uint8_t* v_ptr = aligned + (v_smem - base);
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (bars_smem - base));
  uint64_t* q_full = bars;             // Q of an item landed
  uint64_t* k_full = bars + 1;         // [2] keys of a tile landed
  uint64_t* v_full = bars + 3;         // [2] values landed
  // (a key stage is free when the S product that read it is done, which is what s_full says; a
  // value stage when its PV product is done: o_full.  The producers wait on those: a commit of
  // its own for each cost the issuing warp ≈ 125 cycles a tile)
  uint64_t* s_full = bars + 9;         // [2] S of a tile is in tensor memory
  uint64_t* q_free = bars + 13;        // the item's last S product has read Q
  uint64_t* o_full = bars + 14;        // [2] PV of a tile has been added to O (and its P may be overwritten)
  uint64_t* p_full = bars + 16;        // [2] P of a tile is in tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile uint32_t* failed = tmem_slot + 1;
  float* row_max = reinterpret_cast<float*>(bars + 32);   // [2 tiles][GROUPS][128 rows], then [GROUPS][128] for l

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_items = n_work * nq;
  const int blocks = (int)gridDim.x;

  // the item of this block in round `round`: 0 none is left, 1 an item, 2 a padding item (nothing to do)
  auto get_item = [&](int round, Item& I) -> int {
    const int idx = round * blocks + ((round & 1) ? blocks - 1 - (int)blockIdx.x : (int)blockIdx.x);
    if (idx >= total_items) return 0;
    const int wi = idx / nq;
    I.h = idx - wi * nq;
    const int* w = work + (int64_t)wi * 8;
    I.tok0 = w[1];
    I.ntok = w[2];
    I.pos0 = w[3];
    if (I.ntok == 0) return 2;
    I.table_row = block_table + (int64_t)w[0] * table_stride;
    I.kvh = I.h / (nq / nkv);
    I.pos_last = I.pos0 + I.ntok - 1;
    I.key_lo = (window > 0 && I.pos0 - window + 1 > 0) ? I.pos0 - window + 1 : 0;   // first key any row reads
    I.tile_first = I.key_lo / BLOCK_N;
    I.n_tiles = I.pos_last / BLOCK_N + 1 - I.tile_first;
    return 1;
  };

  const int rows_per_box = page_size < BLOCK_N ? page_size : BLOCK_N;
  const int boxes = BLOCK_N / rows_per_box;              // at most 16: lane b fetches box b of a tile
  // the page of this lane's box of tile `it` of an item, looked up one tile ahead (not yet checked)
  auto lookup = [&](const Item& I, int it) {
    int page = 0;
    if (it < I.n_tiles && lane < boxes) {
      int key = (I.tile_first + it) * BLOCK_N + lane * rows_per_box;
      if (key > I.pos_last) key = I.pos_last;            // past the last key: any page that exists
      if (key < I.key_lo) key = I.key_lo;                // behind the window: pages may have been given back
      page = I.table_row[key / page_size];               // checked where it is used: the load stays in flight
    }
    return page;
  };
  // the work list and the block table are the step's inputs, older than the kernel before this
  // one: the first item's first look-up runs under the set-up below
  Item first_item;
  int first_page = 0;
  const bool producer = warp == 0 || warp == V_WARP;
  if (producer && get_item(0, first_item) == 1) first_page = lookup(first_item, 0);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_free, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&o_full[s], 1);
    }
    mbar_init(&p_full[0], 4 * GROUPS);
    mbar_init(&p_full[1], 4 * GROUPS);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  ls_dependency_wait();                 // q and this step's keys and values come from the kernel before

  if (producer) {
    // ---- producers: warp 0 fetches Q and the key tiles, warp V_WARP the value tiles: a key stage
    // is free two tiles before the value stage of the same tile, and neither waits for the other's ----
    const bool keys = warp == 0;
    uint64_t* free_bar = keys ? s_full : o_full;
    uint64_t* full_bar = keys ? k_full : v_full;
    const uint32_t dst_base = keys ? k_smem : v_smem;
    int gt = 0, j = 0;                  // tiles and items of this block so far
    bool ok = true;
    for (int round = 0; ok; ++round) {
      Item I;
      const int kind = get_item(round, I);
      if (kind == 0) break;
      if (kind == 2) continue;
      int page = round == 0 ? first_page : lookup(I, 0);
      if (keys && lane == 0) {
        // Q is free once the last S product of the item before has read it
        if (j > 0 && (*failed || !mbar_wait(q_free, (uint32_t)(j - 1) & 1u))) {
          *failed = 1;
          ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 810);
        } else {
          mbar_expect_tx(q_full, KV_BYTES);
#pragma unroll
          for (int hh = 0; hh < HALVES; ++hh)
            tma_load_2d(q_smem + hh * HALF_BYTES, &map_q, I.h * D + hh * 64, I.tok0, q_full);
        }
      }
      for (int it = 0; it < I.n_tiles; ++it) {
        const int g = gt + it;
        const int s = g & 1;
        const uint32_t phase = (uint32_t)(g >> 1) & 1u;
        const int c0 = (I.tile_first + it) * BLOCK_N;
        ok = *failed == 0 && mbar_wait(&free_bar[s], phase ^ 1u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          *failed = 1;
          if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 800 + s);
          break;
        }
        if (lane == 0) mbar_expect_tx(&full_bar[s], KV_BYTES);
        __syncwarp();
        if (lane < boxes) {
          if (page < 0 || page >= num_pages) {
            ls_record_fault(err, LS_DEV_PAGE_RANGE, c0 + lane * rows_per_box);
            page = 0;
          }
          const int in_page = ((c0 + lane * rows_per_box) % page_size) / rows_per_box * rows_per_box;
          const int y = ((page * 2 + (keys ? 0 : 1)) * nkv + I.kvh) * page_size + in_page;
#pragma unroll
          for (int hh = 0; hh < HALVES; ++hh)
            tma_load_2d(dst_base + (uint32_t)(s * KV_BYTES + hh * HALF_BYTES + lane * rows_per_box * 128), &map_kv,
                        hh * 64, y, &full_bar[s]);
        }
        page = lookup(I, it + 1);       // after this tile's loads have gone out
      }
      gt += I.n_tiles;
      ++j;
    }
  } else if (warp == 1) {
    // ---- MMA issue: the whole warp walks the loop and one elected lane issues, so that the
    // instructions' operands are the same in every lane and stay in uniform registers (inside a
    // branch of one lane every MMA paid for moving them there) ----
    constexpr uint32_t idesc_s = instr_desc(BLOCK_M, BLOCK_N, false);
    constexpr uint32_t idesc_o = instr_desc(BLOCK_M, D, true);
    const bool issuer = elect_one();
    int gt = 0, j = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      Item I;
      const int kind = get_item(round, I);
      if (kind == 0) break;
      if (kind == 2) continue;
      ok = __all_sync(0xffffffffu, mbar_wait(q_full, (uint32_t)j & 1u));
      auto issue_s = [&](int it) {       // S(it) = Q K(it)^T into the S buffer in turn
        const int g = gt + it;
        const int s = g & 1;
        const uint32_t phase = (uint32_t)(g >> 1) & 1u;
        // (the S buffer is free: the softmax warps had read tile g - 2 before they announced its P,
        // which this warp waited for before the PV product of that tile)
        if (!__all_sync(0xffffffffu, mbar_wait(&k_full[s], phase))) return false;
        fence_after_sync();
        if (issuer) {
#pragma unroll
          for (int k = 0; k < D / UMMA_K; ++k) {
            const uint32_t koff = (uint32_t)((k >> 2) * HALF_BYTES + (k & 3) * UMMA_K * 2);
            umma(tmem_base + S_COL + s * BLOCK_N, desc_k_major(q_smem + koff),
                 desc_k_major(k_smem + s * KV_BYTES + koff), idesc_s, k != 0 ? 1u : 0u);
          }
          umma_commit(&s_full[s]);
          if (it == I.n_tiles - 1) umma_commit(q_free);     // the item's last product with this Q
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int it = 0; it < I.n_tiles && ok; ++it) {
        const int g = gt + it;
        const int s = g & 1;
        const uint32_t phase = (uint32_t)(g >> 1) & 1u;
        if (it + 1 < I.n_tiles) ok = issue_s(it + 1);
        if (!ok) break;
        ok = __all_sync(0xffffffffu, mbar_wait(&p_full[s], phase) && mbar_wait(&v_full[s], phase));
        if (!ok) break;
        fence_after_sync();
        if (issuer) {
#pragma unroll
          for (int k = 0; k < BLOCK_N / UMMA_K; ++k) {
            // P from tensor memory: 16 keys are 8 columns; V: 16 keys are 16 rows of 128 bytes
            const uint64_t b = desc_mn_major(v_smem + s * KV_BYTES + k * UMMA_K * 128, HALF_BYTES);
            umma_ts(tmem_base + O_COL, tmem_base + P_COL + s * P_COLS + k * (UMMA_K / 2), b, idesc_o,
                    (it | k) != 0 ? 1u : 0u);
          }
          umma_commit(&o_full[s]);
        }
        __syncwarp();
      }
      gt += I.n_tiles;
      ++j;
    }
    if (!ok) {
      *failed = 1;
      if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 820);
    }
  } else if (warp < V_WARP) {
    // ---- softmax: GROUPS threads per row (a token, lane `row` of tensor memory): the thread of
    // group g (warps 2 + 4 g .. 5 + 4 g) has keys 32 g .. 32 g + 31 of a tile and the g-th
    // quarter of the head's dimensions ----
    constexpr int HC = BLOCK_N / GROUPS;          // keys of a tile per thread
    constexpr int HD = D / GROUPS;                // output dimensions per thread
    constexpr int ROWS = 128 * GROUPS;            // threads of the softmax
    const int quad = warp & 3;
    const int group = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    // O = sum of P V stays in tensor memory, the MMAs of every tile adding to it, in units of
    // 2^m_ref of its row.  m_ref follows the row's maximum lazily: only when the maximum has
    // grown by more than 8 (a factor 256, which bfloat16 P and float32 sums take easily) is the
    // row of O scaled down and m_ref moved, which after the first tiles hardly ever happens.
    // The quotient O / l does not depend on m_ref.
    constexpr float LAZY = 8.f;
    bool ok = true;
    int gt = 0;

    // A wait that runs out clears `ok`; the loops still run to their ends, skipping the work, so
    // that every thread meets the named barrier of every tile of every item.
    for (int round = 0;; ++round) {
      Item I;
      const int kind = get_item(round, I);
      if (kind == 0) break;
      if (kind == 2) continue;
      const int pos0 = I.pos0, pos_last = I.pos_last, tile_first = I.tile_first, n_tiles = I.n_tiles;
      const int pos = pos0 + row;
      const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
      const int lo_last = (window > 0 && pos_last - window + 1 > 0) ? pos_last - window + 1 : 0;
      float m_ref = -CUDART_INF_F, l_run = 0.f;
      for (int it = 0; it < n_tiles; ++it) {
        const int g = gt + it;
        const int s = g & 1;
        const int c0 = (tile_first + it) * BLOCK_N + group * HC;     // first key of this thread
        if (ok && !mbar_wait(&s_full[s], (uint32_t)(g >> 1) & 1u)) ok = false;
        fence_after_sync();
        // this thread's scores into registers; the buffer is free once all have theirs
        uint32_t sc[HC];
#pragma unroll
        for (int q0 = 0; q0 < HC; q0 += 32) tmem_ld32(lane_base + S_COL + s * BLOCK_N + group * HC + q0, sc + q0);
        tmem_ld_wait();
        // every key of the tile is seen by every row: no masks (uniform over the block)
        const bool full_tile = (tile_first + it) * BLOCK_N + BLOCK_N - 1 <= pos0 && (tile_first + it) * BLOCK_N >= lo_last;
        float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
        if (full_tile) {
#pragma unroll
          for (int jj = 0; jj < HC; jj += 2)
            mx[(jj >> 1) & 3] = max3(mx[(jj >> 1) & 3], __uint_as_float(sc[jj]), __uint_as_float(sc[jj + 1]));
        } else {
          // selects, not branches: a masked score counts as -inf
#pragma unroll
          for (int jj = 0; jj < HC; ++jj) {
            const bool keep = (c0 + jj <= pos) & (c0 + jj >= lo);
            mx[jj & 3] = fmaxf(mx[jj & 3], keep ? __uint_as_float(sc[jj]) : -CUDART_INF_F);
          }
        }
        // the row's maximum is that of its threads
        float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        row_max[(it & 1) * ROWS + group * 128 + row] = tile_max;
        asm volatile("bar.sync 1, %0;" ::"n"(ROWS) : "memory");
#pragma unroll
        for (int o = 0; o < GROUPS; ++o) tile_max = fmaxf(tile_max, row_max[(it & 1) * ROWS + o * 128 + row]);
        // all threads of a row work out the same m_ref from the same numbers
        const float m_new = tile_max * scale_log2;
        const bool move = m_new > m_ref + LAZY;                      // true too for the first key a row sees
        const float factor = move ? ((m_ref == -CUDART_INF_F) ? 0.f : ex2(m_ref - m_new)) : 1.f;
        if (move) m_ref = m_new;
        // this tile's P buffer was read by the PV of two tiles ago (long done); O is scaled only
        // after the PV of the tile before has been added to it
        if (ok && g > 1 && !mbar_wait(&o_full[s], (uint32_t)((g - 2) >> 1) & 1u)) ok = false;
        if (it > 0 && __any_sync(0xffffffffu, move)) {
          if (ok && !mbar_wait(&o_full[(g - 1) & 1], (uint32_t)((g - 1) >> 1) & 1u)) ok = false;
          if (__all_sync(0xffffffffu, ok)) {
            fence_after_sync();
            uint32_t og[HD];
            tmem_ld_cols<HD>(lane_base + O_COL + group * HD, og);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < HD; ++c) og[c] = __float_as_uint(__uint_as_float(og[c]) * factor);
            tmem_st_cols<HD>(lane_base + O_COL + group * HD, og);
          }
        }
        // p = exp2(s * scale - m_ref), rounded to bfloat16, two keys a column, into this thread's
        // columns of the tile's P buffer in tensor memory, from where the PV product takes it as
        // its A operand; the sum in four running sums, folded in a fixed order
        float ps[4] = {0.f, 0.f, 0.f, 0.f};
        const bool dead = m_ref == -CUDART_INF_F;          // nothing seen yet by this row
        const float neg_m = dead ? 0.f : -m_ref;
        uint32_t pk[HC / 2];
        {
          const bool plain = full_tile & !dead;             // uniform over the block but for `dead`
#pragma unroll
          for (int n0 = 0; n0 < HC; n0 += 8) {
            float p[8];
            if (plain) {
#pragma unroll
              for (int jj = 0; jj < 8; jj += 2) {
                p[jj] = __uint_as_float(sc[n0 + jj]);
                p[jj + 1] = __uint_as_float(sc[n0 + jj + 1]);
                fma2(p[jj], p[jj + 1], scale_log2, neg_m);
                p[jj] = ex2(p[jj]);
                p[jj + 1] = ex2(p[jj + 1]);
              }
            } else {
              // every exponential is taken, masked ones of -inf (which is 0): selects, not branches
#pragma unroll
              for (int jj = 0; jj < 8; ++jj) {
                const int key = c0 + n0 + jj;
                const bool keep = (key <= pos) & (key >= lo) & !dead;
                p[jj] = ex2(keep ? fmaf(__uint_as_float(sc[n0 + jj]), scale_log2, neg_m) : -CUDART_INF_F);
              }
            }
            add2(ps[0], ps[1], p[0], p[1]);
            add2(ps[2], ps[3], p[2], p[3]);
            add2(ps[0], ps[1], p[4], p[5]);
            add2(ps[2], ps[3], p[6], p[7]);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) pk[(n0 >> 1) + jj] = pack_bf16(p[2 * jj], p[2 * jj + 1]);
          }
        }
        tmem_st_cols<HC / 2>(lane_base + P_COL + s * P_COLS + group * (HC / 2), pk);
        const float psum = (ps[0] + ps[1]) + (ps[2] + ps[3]);
        // value rows of keys past the last position were never written: they must not be NaN,
        // since P is zero there and the MMA multiplies all the same
        if ((tile_first + it) * BLOCK_N + BLOCK_N - 1 > pos_last) {
          if (ok && !mbar_wait(&v_full[s], (uint32_t)(g >> 1) & 1u)) ok = false;
          if (ok && group < HALVES && (tile_first + it) * BLOCK_N + row > pos_last) {
            uint4* vrow = reinterpret_cast<uint4*>(v_ptr + s * KV_BYTES + group * HALF_BYTES + row * 128);
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) vrow[q8] = make_uint4(0u, 0u, 0u, 0u);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        tmem_st_wait();
        fence_before_sync();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(&p_full[s]);
        l_run = fmaf(l_run, factor, psum);
      }
      // the row's sum is that of its threads (a region of its own: the next item's first tile
      // writes its maxima while a slow thread may still read these)
      float* l_part = row_max + 2 * ROWS;
      l_part[group * 128 + row] = l_run;
      asm volatile("bar.sync 1, %0;" ::"n"(ROWS) : "memory");
      float l_row = l_part[row];                     // the same sum in the same order in each of the row's threads
#pragma unroll
      for (int o = 1; o < GROUPS; ++o) l_row += l_part[o * 128 + row];
      const int g_last = gt + n_tiles - 1;
      if (ok && !mbar_wait(&o_full[g_last & 1], (uint32_t)(g_last >> 1) & 1u)) ok = false;
      if (ok) {
        fence_after_sync();
        uint32_t og[HD];
        tmem_ld_cols<HD>(lane_base + O_COL + group * HD, og);
        tmem_ld_wait();
        fence_before_sync();                         // the next item's first PV overwrites O after its P
        if (row < I.ntok) {
          const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
          __nv_bfloat16* dst = out + ((int64_t)(I.tok0 + row) * nq + I.h) * D + group * HD;
#pragma unroll
          for (int c = 0; c < HD; c += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(og[c]) * inv, __uint_as_float(og[c + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(og[c + 2]) * inv, __uint_as_float(og[c + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(og[c + 4]) * inv, __uint_as_float(og[c + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(og[c + 6]) * inv, __uint_as_float(og[c + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c) = v;
          }
        }
      }
      // (the bar.sync of the next item's first tile, or of its sums, comes before any thread
      // writes this region again)
      gt += n_tiles;
    }
    if (!ok) {
      *failed = 1;
      if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 840 + quad);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}


// ---------------------------------------------------------------------------
// Two query heads of one key head in a block (group sizes that are even).  The two heads'
// tiles Q_A and Q_B (the same 128 tokens) share every key and value tile, which is loaded
// once, and each has a team of eight softmax warps (two threads a row, 64 keys each, read
// from tensor memory in pieces of 32).  Tensor memory: S_A, S_B, O_A, O_B, 128 columns each;
// P (bfloat16, two keys a column) is written over the S it came from, keys 0..63 into the
// first 32 columns and keys 64..127 into columns 64..95, so that a thread only writes over
// scores it has already taken.  The MMAs of one team run while the other team's softmax
// does: S_A, S_B | PV_A, S_A', PV_B, S_B' | ... in this order on the tensor pipe, which
// executes them as issued, so PV_X has read P_X before the next S_X overwrites it.
// A row's arithmetic is that of the kernel above with two threads a row; it depends on the
// row's own position only.
// ---------------------------------------------------------------------------
constexpr int PAIR_THREADS = 19 * 32;
constexpr int PAIR_V_WARP = 18;

template <int HALVES>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
attention_prefill_tc_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                                 __nv_bfloat16* __restrict__ out, const int* __restrict__ work, int n_work,
                                 const int* __restrict__ block_table, int table_stride, int nq, int nkv, int page_size,
                                 int num_pages, int window, float scale_log2, int* err) {
  ls_dependency_trigger();
  constexpr int D = HALVES * 64;
  constexpr int KV_BYTES = HALVES * HALF_BYTES;          // K (or V) of one tile; also one head's Q
  constexpr uint32_t S_COL = 0, O_COL = 2 * BLOCK_N;     // S_X at S_COL + 128 X, O_X at O_COL + 128 X

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;                          // [2 heads]
  const uint32_t k_smem = q_smem + 2 * KV_BYTES;         // [STAGES]
  const uint32_t v_smem = k_smem + STAGES * KV_BYTES;    // [STAGES]
  const uint32_t bars_smem = v_smem + STAGES * KV_BYTES;
  uint8_t* v_ptr = aligned + (v_smem - base);
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (bars_smem - base));
  uint64_t* q_full = bars;             // both heads' Q of an item landed
  uint64_t* k_full = bars + 1;         // [2] keys of a tile landed
  uint64_t* v_full = bars + 3;         // [2] values landed
  uint64_t* k_free = bars + 5;         // [2] both S products have read the stage
  uint64_t* v_free = bars + 7;         // [2] both PV products have read the stage
  uint64_t* s_full = bars + 9;         // [2 teams] S of a tile is in tensor memory
  uint64_t* p_full = bars + 11;        // [2 teams] P of a tile is in tensor memory
  uint64_t* o_full = bars + 13;        // [2 teams] PV of a tile has been added to O
  uint64_t* q_free = bars + 15;        // the item's last S product has read Q
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile uint32_t* failed = tmem_slot + 1;
  float* team_mem = reinterpret_cast<float*>(bars + 32);   // per team: maxima [2][2][128], then sums [4][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pairs = nq >> 1;
  const int total_items = n_work * pairs;
  const int blocks = (int)gridDim.x;

  // the item of this block in round `round`: 0 none is left, 1 an item, 2 a padding item (nothing to do);
  // I.h is the first head of the pair
  auto get_item = [&](int round, Item& I) -> int {
    const int idx = round * blocks + ((round & 1) ? blocks - 1 - (int)blockIdx.x : (int)blockIdx.x);
    if (idx >= total_items) return 0;
    const int wi = idx / pairs;
    I.h = 2 * (idx - wi * pairs);
    const int* w = work + (int64_t)wi * 8;
    I.tok0 = w[1];
    I.ntok = w[2];
    I.pos0 = w[3];
    if (I.ntok == 0) return 2;
    I.table_row = block_table + (int64_t)w[0] * table_stride;
    I.kvh = I.h / (nq / nkv);
    I.pos_last = I.pos0 + I.ntok - 1;
    I.key_lo = (window > 0 && I.pos0 - window + 1 > 0) ? I.pos0 - window + 1 : 0;
    I.tile_first = I.key_lo / BLOCK_N;
    I.n_tiles = I.pos_last / BLOCK_N + 1 - I.tile_first;
    return 1;
  };

  const int rows_per_box = page_size < BLOCK_N ? page_size : BLOCK_N;
  const int boxes = BLOCK_N / rows_per_box;
  auto lookup = [&](const Item& I, int it) {
    int page = 0;
    if (it < I.n_tiles && lane < boxes) {
      int key = (I.tile_first + it) * BLOCK_N + lane * rows_per_box;
      if (key > I.pos_last) key = I.pos_last;
      if (key < I.key_lo) key = I.key_lo;
      page = I.table_row[key / page_size];
    }
    return page;
  };
  Item first_item;
  int first_page = 0;
  const bool producer = warp == 0 || warp == PAIR_V_WARP;
  if (producer && get_item(0, first_item) == 1) first_page = lookup(first_item, 0);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_free, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_free[s], 1);
      mbar_init(&v_free[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 8);
      mbar_init(&o_full[s], 1);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  ls_dependency_wait();

  if (producer) {
    // ---- producers: warp 0 fetches both heads' Q and the key tiles, warp PAIR_V_WARP the value tiles ----
    const bool keys = warp == 0;
    uint64_t* free_bar = keys ? k_free : v_free;
    uint64_t* full_bar = keys ? k_full : v_full;
    const uint32_t dst_base = keys ? k_smem : v_smem;
    int gt = 0, j = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      Item I;
      const int kind = get_item(round, I);
      if (kind == 0) break;
      if (kind == 2) continue;
      int page = round == 0 ? first_page : lookup(I, 0);
      if (keys && lane == 0) {
        if (j > 0 && (*failed || !mbar_wait(q_free, (uint32_t)(j - 1) & 1u))) {
          *failed = 1;
          ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 910);
        } else {
          mbar_expect_tx(q_full, 2 * KV_BYTES);
#pragma unroll
          for (int x = 0; x < 2; ++x)
#pragma unroll
            for (int hh = 0; hh < HALVES; ++hh)
              tma_load_2d(q_smem + x * KV_BYTES + hh * HALF_BYTES, &map_q, (I.h + x) * D + hh * 64, I.tok0, q_full);
        }
      }
      for (int it = 0; it < I.n_tiles; ++it) {
        const int g = gt + it;
        const int s = g & 1;
        const uint32_t phase = (uint32_t)(g >> 1) & 1u;
        const int c0 = (I.tile_first + it) * BLOCK_N;
        ok = *failed == 0 && mbar_wait(&free_bar[s], phase ^ 1u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          *failed = 1;
          if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 900 + s);
          break;
        }
        if (lane == 0) mbar_expect_tx(&full_bar[s], KV_BYTES);
        __syncwarp();
        if (lane < boxes) {
          if (page < 0 || page >= num_pages) {
            ls_record_fault(err, LS_DEV_PAGE_RANGE, c0 + lane * rows_per_box);
            page = 0;
          }
          const int in_page = ((c0 + lane * rows_per_box) % page_size) / rows_per_box * rows_per_box;
          const int y = ((page * 2 + (keys ? 0 : 1)) * nkv + I.kvh) * page_size + in_page;
#pragma unroll
          for (int hh = 0; hh < HALVES; ++hh)
            tma_load_2d(dst_base + (uint32_t)(s * KV_BYTES + hh * HALF_BYTES + lane * rows_per_box * 128), &map_kv,
                        hh * 64, y, &full_bar[s]);
        }
        page = lookup(I, it + 1);
      }
      gt += I.n_tiles;
      ++j;
    }
  } else if (warp == 1) {
    // ---- MMA issue (the whole warp walks the loop, one elected lane issues) ----
    constexpr uint32_t idesc_s = instr_desc(BLOCK_M, BLOCK_N, false);
    constexpr uint32_t idesc_o = instr_desc(BLOCK_M, D, true);
    const bool issuer = elect_one();
    int gt = 0, j = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      Item I;
      const int kind = get_item(round, I);
      if (kind == 0) break;
      if (kind == 2) continue;
      ok = __all_sync(0xffffffffu, mbar_wait(q_full, (uint32_t)j & 1u));
      // S_x(it) = Q_x K(it)^T; the keys are waited for by the first head's product
      auto issue_s = [&](int x, int it) {
        const int g = gt + it;
        const int s = g & 1;
        if (x == 0) {
          if (!__all_sync(0xffffffffu, mbar_wait(&k_full[s], (uint32_t)(g >> 1) & 1u))) return false;
          fence_after_sync();
        }
        if (issuer) {
#pragma unroll
          for (int k = 0; k < D / UMMA_K; ++k) {
            const uint32_t koff = (uint32_t)((k >> 2) * HALF_BYTES + (k & 3) * UMMA_K * 2);
            umma(tmem_base + S_COL + x * BLOCK_N, desc_k_major(q_smem + x * KV_BYTES + koff),
                 desc_k_major(k_smem + s * KV_BYTES + koff), idesc_s, k != 0 ? 1u : 0u);
          }
          umma_commit(&s_full[x]);
          if (x == 1) {
            umma_commit(&k_free[s]);
            if (it == I.n_tiles - 1) umma_commit(q_free);
          }
        }
        __syncwarp();
        return true;
      };
      // O_x += P_x(it) V(it); the values are waited for by the first head's product
      auto issue_pv = [&](int x, int it) {
        const int g = gt + it;
        const int s = g & 1;
        bool got = mbar_wait(&p_full[x], (uint32_t)g & 1u);
        if (x == 0) got = got && mbar_wait(&v_full[s], (uint32_t)(g >> 1) & 1u);
        if (!__all_sync(0xffffffffu, got)) return false;
        fence_after_sync();
        if (issuer) {
#pragma unroll
          for (int k = 0; k < BLOCK_N / UMMA_K; ++k) {
            // 16 keys are 8 columns of P: keys 0..63 at columns 0..31 of S_x, keys 64..127 at 64..95
            const uint32_t pcol = (uint32_t)(k < 4 ? k * 8 : 64 + (k - 4) * 8);
            const uint64_t b = desc_mn_major(v_smem + s * KV_BYTES + k * UMMA_K * 128, HALF_BYTES);
            umma_ts(tmem_base + O_COL + x * 128, tmem_base + S_COL + x * BLOCK_N + pcol, b, idesc_o,
                    (it | k) != 0 ? 1u : 0u);
          }
          umma_commit(&o_full[x]);
          if (x == 1) umma_commit(&v_free[s]);
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_s(0, 0);
      if (ok) ok = issue_s(1, 0);
      for (int it = 0; it < I.n_tiles && ok; ++it) {
        ok = issue_pv(0, it);
        if (ok && it + 1 < I.n_tiles) ok = issue_s(0, it + 1);
        if (ok) ok = issue_pv(1, it);
        if (ok && it + 1 < I.n_tiles) ok = issue_s(1, it + 1);
      }
      gt += I.n_tiles;
      ++j;
    }
    if (!ok) {
      *failed = 1;
      if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 920);
    }
  } else if (warp < PAIR_V_WARP) {
    // ---- softmax: team x = (warp - 2) / 8 has head I.h + x; two threads a row: `sub` has keys
    // 64 sub .. 64 sub + 63 of a tile (read in pieces of 32) and half of the head's dimensions ----
    constexpr int HC = 32;                        // scores in registers at a time
    const int team = (warp - 2) >> 3;
    const int sub = ((warp - 2) >> 2) & 1;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_col = lane_base + S_COL + team * BLOCK_N;
    const uint32_t o_col = lane_base + O_COL + team * 128 + sub * (D / 2);
    float* tmax = team_mem + team * 1024;         // [parity][sub][128]: the two threads of a row exchange their maxima
    float* l_part = tmax + 512;                   // [quarter][128]
    constexpr float LAZY = 8.f;
    bool ok = true;
    int gt = 0;
    // A wait that runs out clears `ok`; the loops still run to their ends, skipping the work, so
    // that every thread meets the named barriers of every tile of every item.
    for (int round = 0;; ++round) {
      Item I;
      const int kind = get_item(round, I);
      if (kind == 0) break;
      if (kind == 2) continue;
      const int pos0 = I.pos0, pos_last = I.pos_last, tile_first = I.tile_first, n_tiles = I.n_tiles;
      const int pos = pos0 + row;
      const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
      const int lo_last = (window > 0 && pos_last - window + 1 > 0) ? pos_last - window + 1 : 0;
      // the sum of a row's weights is kept per quarter of a tile's keys (32 sub .. + 31), as the
      // kernel with four threads a row keeps it, so that both give the same bits
      float m_ref = -CUDART_INF_F, l_run[2] = {0.f, 0.f};
      for (int it = 0; it < n_tiles; ++it) {
        const int g = gt + it;
        const int s = g & 1;                       // stage of the tile's keys and values
        const int c0 = (tile_first + it) * BLOCK_N + sub * 64;        // first key of this thread
        if (ok && !mbar_wait(&s_full[team], (uint32_t)g & 1u)) ok = false;
        fence_after_sync();
        const bool full_tile = (tile_first + it) * BLOCK_N + BLOCK_N - 1 <= pos0 && (tile_first + it) * BLOCK_N >= lo_last;
        // ---- the row's maximum over the tile ----
        float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int piece = 0; piece < 2; ++piece) {
          uint32_t sc[HC];
          tmem_ld32(s_col + sub * 64 + piece * HC, sc);
          tmem_ld_wait();
          if (full_tile) {
#pragma unroll
            for (int jj = 0; jj < HC; jj += 2)
              mx[(jj >> 1) & 3] = max3(mx[(jj >> 1) & 3], __uint_as_float(sc[jj]), __uint_as_float(sc[jj + 1]));
          } else {
            // selects, not branches: a masked score counts as -inf
#pragma unroll
            for (int jj = 0; jj < HC; ++jj) {
              const int key = c0 + piece * HC + jj;
              const bool keep = (key <= pos) & (key >= lo);
              mx[jj & 3] = fmaxf(mx[jj & 3], keep ? __uint_as_float(sc[jj]) : -CUDART_INF_F);
            }
          }
        }
        float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        const int par = it & 1;
        tmax[par * 256 + sub * 128 + row] = tile_max;
        if (team == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
        else asm volatile("bar.sync 2, 256;" ::: "memory");
        tile_max = fmaxf(tmax[par * 256 + row], tmax[par * 256 + 128 + row]);
        // both threads of a row work out the same m_ref from the same numbers
        const float m_new = tile_max * scale_log2;
        const bool move = m_new > m_ref + LAZY;                      // true too for the first key a row sees
        const float factor = move ? ((m_ref == -CUDART_INF_F) ? 0.f : ex2(m_ref - m_new)) : 1.f;
        if (move) m_ref = m_new;
        // O is scaled only after the PV of the tile before has been added to it (and before this
        // tile's P is announced, so before the PV of this tile)
        if (it > 0 && __any_sync(0xffffffffu, move)) {
          if (ok && !mbar_wait(&o_full[team], (uint32_t)(g - 1) & 1u)) ok = false;
          if (__all_sync(0xffffffffu, ok)) {
            fence_after_sync();
#pragma unroll
            for (int piece = 0; piece < D / 64; ++piece) {            // this thread's half of the row, 32 columns at a time
              uint32_t og[32];
              tmem_ld32(o_col + piece * 32, og);
              tmem_ld_wait();
#pragma unroll
              for (int c = 0; c < 32; ++c) og[c] = __float_as_uint(__uint_as_float(og[c]) * factor);
              tmem_st32(o_col + piece * 32, og);
            }
          }
        }
        // ---- p = exp2(s * scale - m_ref), rounded to bfloat16, two keys a column, written over
        // scores this thread has already taken ----
        const bool dead = m_ref == -CUDART_INF_F;          // nothing seen yet by this row
        const float neg_m = dead ? 0.f : -m_ref;
        const bool plain = full_tile & !dead;               // uniform over the block but for `dead`
#pragma unroll
        for (int piece = 0; piece < 2; ++piece) {
          uint32_t sc[HC];
          tmem_ld32(s_col + sub * 64 + piece * HC, sc);
          tmem_ld_wait();
          uint32_t pk[HC / 2];
          float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int n0 = 0; n0 < HC; n0 += 8) {
            float p[8];
            if (plain) {
#pragma unroll
              for (int jj = 0; jj < 8; jj += 2) {
                p[jj] = __uint_as_float(sc[n0 + jj]);
                p[jj + 1] = __uint_as_float(sc[n0 + jj + 1]);
                fma2(p[jj], p[jj + 1], scale_log2, neg_m);
                p[jj] = ex2(p[jj]);
                p[jj + 1] = ex2(p[jj + 1]);
              }
            } else {
              // every exponential is taken, masked ones of -inf (which is 0): selects, not branches
#pragma unroll
              for (int jj = 0; jj < 8; ++jj) {
                const int key = c0 + piece * HC + n0 + jj;
                const bool keep = (key <= pos) & (key >= lo) & !dead;
                p[jj] = ex2(keep ? fmaf(__uint_as_float(sc[n0 + jj]), scale_log2, neg_m) : -CUDART_INF_F);
              }
            }
            add2(ps[0], ps[1], p[0], p[1]);
            add2(ps[2], ps[3], p[2], p[3]);
            add2(ps[0], ps[1], p[4], p[5]);
            add2(ps[2], ps[3], p[6], p[7]);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) pk[(n0 >> 1) + jj] = pack_bf16(p[2 * jj], p[2 * jj + 1]);
          }
          tmem_st16(s_col + sub * 64 + piece * (HC / 2), pk);
          l_run[piece] = fmaf(l_run[piece], factor, (ps[0] + ps[1]) + (ps[2] + ps[3]));
        }
        // value rows of keys past the last position were never written: they must not be NaN,
        // since P is zero there and the MMA multiplies all the same
        if ((tile_first + it) * BLOCK_N + BLOCK_N - 1 > pos_last) {
          if (ok && !mbar_wait(&v_full[s], (uint32_t)(g >> 1) & 1u)) ok = false;
          if (ok && sub < HALVES && (tile_first + it) * BLOCK_N + row > pos_last) {
            uint4* vrow = reinterpret_cast<uint4*>(v_ptr + s * KV_BYTES + sub * HALF_BYTES + row * 128);
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) vrow[q8] = make_uint4(0u, 0u, 0u, 0u);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        tmem_st_wait();
        fence_before_sync();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(&p_full[team]);
      }
      // ---- the item's end: the row's sum is that of its four quarters in order; each thread
      // writes half of the row out ----
      l_part[(sub * 2) * 128 + row] = l_run[0];
      l_part[(sub * 2 + 1) * 128 + row] = l_run[1];
      if (team == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
      else asm volatile("bar.sync 2, 256;" ::: "memory");
      float l_row = l_part[row];
#pragma unroll
      for (int o = 1; o < 4; ++o) l_row += l_part[o * 128 + row];
      const int g_last = gt + n_tiles - 1;
      if (ok && !mbar_wait(&o_full[team], (uint32_t)g_last & 1u)) ok = false;
      if (ok) {
        fence_after_sync();
        const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
        __nv_bfloat16* dst = out + ((int64_t)(I.tok0 + row) * nq + I.h + team) * D + sub * (D / 2);
#pragma unroll
        for (int piece = 0; piece < D / 64; ++piece) {
          uint32_t og[32];
          tmem_ld32(o_col + piece * 32, og);
          tmem_ld_wait();
          if (row < I.ntok) {
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(og[c]) * inv, __uint_as_float(og[c + 1]) * inv);
              v.y = pack_bf16(__uint_as_float(og[c + 2]) * inv, __uint_as_float(og[c + 3]) * inv);
              v.z = pack_bf16(__uint_as_float(og[c + 4]) * inv, __uint_as_float(og[c + 5]) * inv);
              v.w = pack_bf16(__uint_as_float(og[c + 6]) * inv, __uint_as_float(og[c + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + piece * 32 + c) = v;
            }
          }
        }
        fence_before_sync();                         // the next item's first PV overwrites O after its P
      }
      // the sums are read before any thread writes them for the next item
      if (team == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
      else asm volatile("bar.sync 2, 256;" ::: "memory");
      gt += n_tiles;
    }
    if (!ok) {
      *failed = 1;
      if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 940 + quad);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
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

bool encode(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t rows, uint32_t box_rows) {
  EncodeTiled enc = encode_fn();
  if (enc == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)inner * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

// 0: a head a block always; 1: two heads of a key head a block where that pays; 2: wherever the group is even
int pair_heads = 1;

template <int HALVES>
int launch(const CUtensorMap& map_q, const CUtensorMap& map_kv, void* out, const int* work, int n_work,
           const int* block_table, int table_stride, int nq, int nkv, int page_size, int num_pages, int window,
           float scale, int* err, cudaStream_t stream) {
  constexpr int KV_BYTES = HALVES * HALF_BYTES;
  const size_t smem = (size_t)KV_BYTES * (1 + 2 * STAGES) + 256 + 3 * 128 * GROUPS * 4 + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_tc_kernel<HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return LS_E_SMEM;
    configured = true;
  }
  // two heads of a key head in a block where the group size is even and there are items enough
  // to fill the device one and a half times over (with fewer, the longest item would set the
  // time: a prompt of 2,048 tokens and 16 heads is 128 pairs, the longest of 16 double tiles)
  if (pair_heads && (nq / nkv) % 2 == 0 &&
      (pair_heads > 1 || 2LL * n_work * (nq / 2) >= 3LL * sm_count())) {
    const size_t pair_smem = (size_t)KV_BYTES * (2 + 2 * STAGES) + 256 + 2 * 1024 * 4 + 1024;
    static bool pair_configured = false;
    if (!pair_configured) {
      if (cudaFuncSetAttribute(attention_prefill_tc_pair_kernel<HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)pair_smem) != cudaSuccess)
        return LS_E_SMEM;
      pair_configured = true;
    }
    const long long pair_items = (long long)n_work * (nq / 2);
    const int pair_blocks = pair_items < sm_count() ? (int)pair_items : sm_count();
    LS_COUNT(LS_K_ATTENTION_PREFILL_TC), ls_launch(attention_prefill_tc_pair_kernel<HALVES>, dim3(pair_blocks), PAIR_THREADS, pair_smem, stream, map_q, map_kv,
              (__nv_bfloat16*)out, work, n_work, block_table, table_stride, nq, nkv, page_size, num_pages, window,
              scale * 1.4426950408889634f, err);
    return ls_launch_status();
  }
  // a block per SM (its shared memory and its 512 columns of tensor memory fill one), or fewer items
  const long long items = (long long)n_work * nq;
  const int blocks = items < sm_count() ? (int)items : sm_count();
  LS_COUNT(LS_K_ATTENTION_PREFILL_TC), ls_launch(attention_prefill_tc_kernel<HALVES>, dim3(blocks), THREADS, smem, stream, map_q, map_kv, (__nv_bfloat16*)out, work, n_work,
            block_table, table_stride, nq, nkv, page_size, num_pages, window, scale * 1.4426950408889634f, err);
  return ls_launch_status();
}

}  // namespace

LS_API int ls_attention_prefill_tc_tile_tokens() { return BLOCK_M; }
LS_API void ls_set_attention_prefill_pairs(int mode) { pair_heads = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }

// q, out: [tokens, nq * d] bfloat16; pages [num_pages, 2, nkv, page_size, d]; d 64 or 128; page
// sizes 8, 16, 32, 64, 128.  Work items as for ls_attention_tile with up to 128 tokens each
// (splits and slots are not used).  Returns LS_E_SIZE or LS_E_ALIGN for anything else, having
// launched nothing.
LS_API int ls_attention_prefill_tc(const void* q, const void* pages, void* out, int tokens, const int* work,
                                   int n_work, const int* block_table, int table_stride, int nq, int nkv, int d,
                                   int page_size, int num_pages, int window, float scale, int* err,
                                   cudaStream_t stream) {
  if (n_work <= 0 || tokens <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv || n_work > 65535) return LS_E_SIZE;
  if (d != 64 && d != 128) return LS_E_SIZE;
  if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return LS_E_SIZE;
  const int64_t rows = (int64_t)num_pages * 2 * nkv * page_size;
  if (rows > 2147483647LL) return LS_E_SIZE;
  if (((uintptr_t)pages & 127) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15)) return LS_E_ALIGN;
  CUtensorMap map_q, map_kv;
  if (!encode(&map_q, q, (uint64_t)nq * d, (uint64_t)tokens, BLOCK_M)) return LS_E_SIZE;
  if (!encode(&map_kv, pages, (uint64_t)d, (uint64_t)rows, page_size < BLOCK_N ? page_size : BLOCK_N)) return LS_E_SIZE;
  if (d == 64)
    return launch<1>(map_q, map_kv, out, work, n_work, block_table, table_stride, nq, nkv, page_size, num_pages,
                     window, scale, err, stream);
  return launch<2>(map_q, map_kv, out, work, n_work, block_table, table_stride, nq, nkv, page_size, num_pages,
                   window, scale, err, stream);
}

LS_API const char* ls_constants_attention_prefill_tc() {
  static char buf[256];
  static const LsConstant c[] = {{"attention_prefill_tc.queries", BLOCK_M}, {"attention_prefill_tc.keys", BLOCK_N},
                                 {"attention_prefill_tc.softmax_threads_per_row", GROUPS}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}
