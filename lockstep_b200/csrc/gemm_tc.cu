// C[T, N] = X[T, K] * W[N, K]^T in bfloat16 on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory, operands staged by TMA).
//
// Orientation: up to 128 tokens, the weight tile is the MMA's M side (128 rows of
// W) and the tokens are its N side (16..128 per tile), so a batch of one decoded
// token wastes no rows of the MMA; more tokens are the M side themselves
// (gemm_tc_rows_kernel: 256 a tile on a pair of blocks, tcgen05 cta_group::2, each
// block with its 128 tokens and half of the weight rows), whose outputs then lie
// side by side in a thread.
// Either way an output element is the same dot product, accumulated in the same
// order, and the two give the same bits.  A block walks its share of K in
// ascending 64-element blocks.  Where the weight gives too few tiles to occupy
// the device (few rows of tiles, deep K) and the tokens are few, K is cut into
// shares run by the blocks of one thread-block cluster, and the shares' partial
// tiles are summed in ascending share order through distributed shared memory
// (pushed with st.async for few tokens, read after a cluster barrier for more);
// with many tokens one block walks the shares of its tile one after the other.
// The number of shares is a function of the weight's shape alone
// (ls_gemm_tc_k_shares), so an output element is the same sum whatever the batch.
//
// Roles inside a block (192 threads; 320 with eight epilogue warps): warp 0 issues
// TMA loads into a ring of shared-memory stages, warp 1 walks the loop of the MMAs
// whole and one elected lane of it issues them and commits stages back, warps
// 2.. read the accumulator from tensor memory and write the epilogue:
//   0 store     C[t, n]  = acc                      (bfloat16 or float32)
//   1 residual  C[t, n] += acc                      (float32, in place)
//   2 silu-mul  C[t, n]  = silu(acc_gate) * acc_up  (W holds gate rows [0, N)
//                                                    and up rows [N, 2N); silu_mul())
//   3 q/k/v     the rows of W are q, k and v heads: each head of a token is
//               rounded to bfloat16 and goes where ls_qkv_head_store puts it (q
//               normed and rotated, k normed and rotated into its cache page, v
//               copied there); few tokens only
// Every wait on a barrier is bounded; a wait that runs out records
// LS_DEV_WAIT_TIMEOUT in the error word and the block winds down (waits for its
// own copies in flight, frees its tensor memory, returns).
#include <cuda.h>

#include "common.cuh"
#include "rope.cuh"
#include "tc_common.cuh"

// Into how many shares K is cut for a weight of N rows and depth K: a function of the
// weight's shape alone.  With few tokens a block streams one share of one row tile, a block
// to an SM, and the device takes the blocks in rounds of 148 (its number of SMs: a constant
// of this rule and not a query, so that the sums are the same on any device).  A round costs
// the share's depth in 64-element blocks plus a fixed part worth 22 of them (the chain of
// latencies of a block and the token rows it norms again; measured on the gate/up weights of
// the 4B and 8B sizes, where 10 chose three shares and lost 14 us a layer at 8B).  The rule
// takes the number of shares (each at least four blocks deep, at most 8, the portable cluster
// size) with the smallest rounds x (depth / shares + 22), the fewest shares among equals.
#define LS_SHARE_RULE_BLOCKS 148        // blocks of a round
#define LS_SHARE_RULE_FIXED 22          // fixed cost of a round, in 64-element blocks of K
#define LS_SHARE_RULE_MIN_DEPTH 4       // a share is at least this many blocks deep
#define LS_SHARE_RULE_MAX_SHARES 8      // the portable cluster size
LS_API int ls_gemm_tc_k_shares(int N, int K) {
  const long long tiles = (N + 127) / 128;
  const long long kb = (K + 63) / 64;
  const long long fixed = LS_SHARE_RULE_FIXED, round = LS_SHARE_RULE_BLOCKS;
  long long most = kb / LS_SHARE_RULE_MIN_DEPTH;
  if (most > LS_SHARE_RULE_MAX_SHARES) most = LS_SHARE_RULE_MAX_SHARES;
  long long best = 1;
  long long best_cost = ((tiles + round - 1) / round) * (kb + fixed);        // cost x shares, compared as cross products
  for (long long s = 2; s <= most; ++s) {
    const long long cost = ((tiles * s + round - 1) / round) * (kb + fixed * s);
    if (cost * best < best_cost * s) {
      best = s;
      best_cost = cost;
    }
  }
  return (int)best;
}

namespace {

constexpr int BM = 128;           // rows of W per tile (MMA M)
constexpr int BK = 64;            // K elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;

// silu(a) * up as every epilogue of this file computes it: the exponential and the reciprocal
// are the hardware's approximations (within 2 ulp each; the product is rounded to bfloat16 by
// its one user).  With expf and a division the silu-mul epilogue of a 128 x 128 tile took as
// long as the tile's MMAs.  Far below zero the result is -0 * up, as with the exact form.
__device__ __forceinline__ float silu_mul(float a, float up) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a * -1.4426950408889634f));
  return __fdividef(a, 1.0f + e) * up;
}

__host__ __device__ constexpr int tmem_cols(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

template <int BN, int EPI>
struct Shape {
  static constexpr int A_TILES = EPI == 2 ? 2 : 1;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
  static constexpr int STAGES_FIT = (200 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 10 ? 10 : STAGES_FIT;
  static constexpr int REGION_COLS = A_TILES * BN;      // one accumulator (gate and up for silu-mul)
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
};

template <int EPI, typename TC>
__device__ __forceinline__ void epilogue_store(TC* c, float a, float up) {
  if (EPI == 0) {
    *c = ls_from_float<TC>(a);
  } else if (EPI == 1) {
    *c = ls_from_float<TC>(ls_to_float<TC>(*c) + a);
  } else {
    *c = ls_from_float<TC>(silu_mul(a, up));
  }
}

__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

constexpr int MAX_SHARES = 8;

// K is cut into `shares` shares of kb_per_share 64-element blocks.  An output
// element is  ((0 + p_0) + p_1) + ... + p_{shares-1}  with p_r the float32
// accumulation of share r in ascending k.  The shares of a tile run in the
// `shares` blocks of a cluster (gemm_tc_few_kernel for a tile of 16 or 32 tokens,
// this kernel for 64 or 128) or one after the other in one persistent block
// (gemm_tc_walk_kernel); all three give the same bits.
//
// This kernel: every block leaves its partial tile in its own shared memory, the
// cluster meets at a barrier, and block r folds the columns c with c % shares == r,
// reading all shares through distributed shared memory.
constexpr int NORM_X_BYTES = 64 * 1024;        // most shared memory a normed token operand may take

template <int BN, int EPI>
struct ClusterShape {
  static constexpr int A_TILES = EPI == 2 ? 2 : 1;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
  static constexpr int RING = 200 * 1024;
  static constexpr int STAGES_FIT = RING / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 10 ? 10 : STAGES_FIT;
  static constexpr int REGION_COLS = A_TILES * BN;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
  static_assert((size_t)STAGES * STAGE_BYTES >= (size_t)REGION_COLS * BM * 4, "no room to stage the partial tile");
};

struct NormArgs {
  const float* h;          // [src_rows, K] float32
  const int* row_index;    // rows of h to take, or null for rows 0 .. T-1
  const void* gain;        // [K]
  int gain_bf16;           // element type of gain: 1 bfloat16, 0 float32
  int src_rows;
  float eps;
};

template <int BN, int EPI, typename TC>
__global__ void __launch_bounds__(192, 1)
gemm_tc_cluster_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                       TC* __restrict__ C, int T, int N, int K, int64_t ldc,
                       int kb_per_share, int shares, int* err) {
  using S = ClusterShape<BN, EPI>;
  ls_dependency_trigger();                      // set-up and the weight loads run while the previous
                                                // kernel drains; its results are touched after the wait
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (size_t)S::STAGES * S::STAGE_BYTES);
  uint64_t* full = bars;                        // [STAGES] operands landed
  uint64_t* empty = bars + S::STAGES;           // [STAGES] MMAs have read the stage
  uint64_t* acc_full = bars + 2 * S::STAGES;    // [1] the accumulator is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* failed = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM;
  const int t0 = blockIdx.y * BN;
  const int total_kb = (K + BK - 1) / BK;
  const int kb_begin = (int)blockIdx.z * kb_per_share;          // this block's share of K
  int kb_end = kb_begin + kb_per_share;
  if (kb_end > total_kb) kb_end = total_kb;
  const int num_kb = kb_end - kb_begin;
  constexpr uint32_t ACC_COLS = (uint32_t)tmem_cols(S::REGION_COLS);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(ACC_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  float first_old = 0.f;        // residual epilogue: the old value of the first column this block folds
  if (warp == 0) {
    if (lane == 0) {
      // the weights do not depend on the previous kernel; the token operand read by TMA does:
      // the first round of the ring takes its weights before the wait and its tokens after
      const int first_round = num_kb < S::STAGES ? num_kb : S::STAGES;
      for (int kb = 0; kb < first_round; ++kb) {
        const uint32_t stage = base + (uint32_t)kb * S::STAGE_BYTES;
        mbar_expect_tx(&full[kb], S::STAGE_BYTES);
        const int kx = (kb_begin + kb) * BK;
        tma_load_2d(stage, &map_w, kx, n0, &full[kb]);
        if (EPI == 2) tma_load_2d(stage + A_BYTES, &map_w, kx, N + n0, &full[kb]);
      }
      ls_dependency_wait();
      for (int kb = 0; kb < first_round; ++kb)
        tma_load_2d(base + (uint32_t)kb * S::STAGE_BYTES + S::A_TILES * A_BYTES, &map_x, (kb_begin + kb) * BK, t0,
                    &full[kb]);
      int issued = first_round;
      for (int kb = first_round; kb < num_kb; ++kb) {
        const int s = kb % S::STAGES;
        const uint32_t phase = (uint32_t)(kb / S::STAGES) & 1u;
        if (*failed || !mbar_wait(&empty[s], phase ^ 1u)) {
          *failed = 1;
          ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 100 + s);
          break;
        }
        const uint32_t stage = base + (uint32_t)s * S::STAGE_BYTES;
        mbar_expect_tx(&full[s], S::STAGE_BYTES);
        const int kx = (kb_begin + kb) * BK;
        tma_load_2d(stage, &map_w, kx, n0, &full[s]);
        if (EPI == 2) tma_load_2d(stage + A_BYTES, &map_w, kx, N + n0, &full[s]);
        tma_load_2d(stage + S::A_TILES * A_BYTES, &map_x, kx, t0, &full[s]);
        issued = kb + 1;
      }
      if (*failed) {
        // wait (bounded) for the copies still in flight before the block exits
        const int first = issued > S::STAGES ? issued - S::STAGES : 0;
        for (int kb = first; kb < issued; ++kb)
          mbar_wait(&full[kb % S::STAGES], (uint32_t)(kb / S::STAGES) & 1u);
      }
    }
  } else if (warp == 1) {
    // the whole warp walks the loop and one elected lane issues: the instructions' operands
    // are then the same in every lane and need no move into uniform registers per MMA
    constexpr uint32_t idesc = instr_desc(BM, BN);
    const bool issuer = elect_one();
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % S::STAGES;
      const uint32_t phase = (uint32_t)(kb / S::STAGES) & 1u;
      ok = __all_sync(0xffffffffu, !*failed && mbar_wait(&full[s], phase));
      if (!ok) {
        *failed = 1;
        if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 200 + s);
        break;
      }
      fence_after_sync();
      const uint32_t stage = base + (uint32_t)s * S::STAGE_BYTES;
      const uint64_t adesc = desc_k_major(stage), udesc = desc_k_major(stage + A_BYTES);
      const uint64_t bdesc = desc_k_major(stage + S::A_TILES * A_BYTES);
      if (issuer) {
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
          umma(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, acc);
          if (EPI == 2) umma(tmem_base + BN, udesc + 2 * k, bdesc + 2 * k, idesc, acc);
        }
        if (kb + S::STAGES < num_kb) umma_commit(&empty[s]);     // only a stage that is filled again
      }
      __syncwarp();
    }
    if (ok && issuer) umma_commit(acc_full);
    __syncwarp();
  } else {
    // epilogue warps: warp w may touch tensor-memory lanes 32*(w%4) .. +32
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    ls_dependency_wait();
    if (EPI == 1 && (int)blockIdx.z < BN && t0 + (int)blockIdx.z < T && n0 + row < N)
      first_old = ls_to_float<TC>(C[(int64_t)(t0 + (int)blockIdx.z) * ldc + n0 + row]);   // in flight during the products
    bool ok = mbar_wait(acc_full, 0);
    if (!ok) {
      *failed = 1;
      if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 300 + quad);
    }
    ok = __all_sync(0xffffffffu, ok);
    fence_after_sync();
    if (ok) {
      // leave this share's partial tile in shared memory: part[column][row], float32
      float* part = reinterpret_cast<float*>(aligned);
#pragma unroll 1
      for (int c0 = 0; c0 < S::REGION_COLS; c0 += 16) {
        uint32_t g[16];
        tmem_ld16(lane_base + c0, g);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) part[(c0 + j) * BM + row] = __uint_as_float(g[j]);
      }
    }
  }
  // all shares have left their partials; each block folds the columns c with
  // c % shares == its rank, reading every share in ascending order
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (warp >= 2 && !*failed) {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int n = n0 + row;
    uint32_t peer[MAX_SHARES];
#pragma unroll
    for (int r = 0; r < MAX_SHARES; ++r)
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[r]) : "r"(base), "r"(r < shares ? r : 0));
    // FOLD columns at a time: their shares' values (and the old values of a residual) are all
    // asked for before any is used, so that a block pays a few trips through the cluster's
    // shared memory and not one per column
    constexpr int FOLD = 4;
    for (int c0 = (int)blockIdx.z; c0 < BN; c0 += FOLD * shares) {
      float vg[FOLD][MAX_SHARES], vu[FOLD][MAX_SHARES], before[FOLD];
#pragma unroll
      for (int f = 0; f < FOLD; ++f) {
        const int c = c0 + f * shares;
        const bool live = c < BN && t0 + c < T;
        const uint32_t off_g = (uint32_t)((c * BM + row) * 4), off_u = (uint32_t)(((BN + c) * BM + row) * 4);
#pragma unroll
        for (int r = 0; r < MAX_SHARES; ++r) {
          vg[f][r] = (live && r < shares) ? ld_cluster_f32(peer[r] + off_g) : 0.f;
          if (EPI == 2) vu[f][r] = (live && r < shares) ? ld_cluster_f32(peer[r] + off_u) : 0.f;
        }
        before[f] = 0.f;
        if (EPI == 1 && live && n < N)
          before[f] = c == (int)blockIdx.z ? first_old : ls_to_float<TC>(C[(int64_t)(t0 + c) * ldc + n]);
      }
#pragma unroll
      for (int f = 0; f < FOLD; ++f) {
        const int c = c0 + f * shares;
        if (c >= BN || t0 + c >= T) break;
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int r = 0; r < MAX_SHARES; ++r) {
          if (r < shares) {
            g += vg[f][r];
            if (EPI == 2) u += vu[f][r];
          }
        }
        if (n < N) {
          TC* cp = C + (int64_t)(t0 + c) * ldc + n;
          if (EPI == 1) {
            *cp = ls_from_float<TC>(before[f] + g);
          } else {
            epilogue_store<EPI, TC>(cp, g, u);
          }
        }
      }
    }
  }
  // no block may leave while a peer still reads its partial
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
  fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Few tokens (a tile of 16 or 32): the decode step's products.  The same shares
// in the blocks of a cluster, but nothing waits at a cluster barrier for the
// sums.  A block that has its share's tile pushes every column straight from
// registers into the shared memory of the block that folds that column (column
// c belongs to rank c % shares) with stores that count their bytes on that
// block's barrier (st.async); a block folds as soon as the bytes of all shares
// have landed, a block with no column to fold does not wait at all, and either
// may leave at
// once, since nobody reads its memory.  The ring is as deep as the share (all
// weights of a block are in flight before the previous kernel has ended), and
// with NORM the token operand is not read by TMA but made here from float32 rows,
// x[t, :] = h[row(t), :] * rsqrt(mean(h^2) + eps) * gain rounded to bfloat16, with
// exactly the arithmetic of rmsnorm_kernel, so that the fused and the separate
// form give the same bits; the epilogue warps do it, two rows of a warp at a time
// with all their loads in flight together, the gain fetched before the wait on
// the previous kernel.  Sums and their order are those of the other two kernels.
// ---------------------------------------------------------------------------
constexpr int MAX_STAGES = 12;

struct FewLayout {
  int stages;            // depth of the ring
  int slots;             // columns one block folds: ceil(BN / shares)
  uint32_t x_off;        // NORM: normed rows [kb][BN][128 B], from the aligned base
  uint32_t recv_off;     // received partials [share][slot][part][128] float32
  uint32_t head_off;     // q/k/v epilogue: folded columns [slot][128] bfloat16
  uint32_t bars_off;     // barriers and words
  uint32_t smem;         // dynamic shared memory of the launch
};

__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, int rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
// A float32 into a peer's shared memory that counts itself (4 bytes) on the peer's barrier
// when it has landed: no fence and no separate arrival follow the pushes.
__device__ __forceinline__ void st_async_f32(uint32_t cluster_addr, float v, uint32_t cluster_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(cluster_addr),
               "r"(__float_as_uint(v)), "r"(cluster_bar)
               : "memory");
}
// the limit is four times that of a block's own waits: a peer that ran into its own limit
// is given up on later than that
__device__ __forceinline__ bool mbar_wait_long(uint64_t* bar, uint32_t parity) {
  return mbar_wait_for(bar, parity, 4 * WAIT_CYCLES);
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The gain of a share's columns as one lane needs it (groups k_lo/4 + lane + 32 j), fetched
// before the wait on the previous kernel: a weight, and the one access of the norm that
// goes to device memory.
constexpr int GAIN_KEEP = 4;      // float4 groups per lane kept in registers (a share of 512 columns)

__device__ __forceinline__ float4 load_gain4(const NormArgs& norm, int g) {
  typedef __nv_bfloat16 bf16;
  if (norm.gain_bf16) {
    const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(norm.gain) + 4 * g);
    const __nv_bfloat162 g01 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 g23 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__bfloat162float(g01.x), __bfloat162float(g01.y), __bfloat162float(g23.x),
                       __bfloat162float(g23.y));
  }
  return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(norm.gain) + 4 * g);
}

// Rows t_a and t_b (t_b < 0: none) of the token tile, normed and rounded, written into the
// swizzled operand layout: the arithmetic of rmsnorm_kernel (lane l sums the float4 groups
// l, l + 32, ... in order, lanes by an xor tree), with the loads of both rows issued together.
template <int BN>
__device__ __forceinline__ void normed_rows_to_smem(const NormArgs& norm, const float4* gain_kept,
                                                    uint8_t* x_region, int t_a, int t_b, int t0, int K,
                                                    int k_lo, int k_hi, int num_kb, int lane, int* err) {
  constexpr int U = 8;                               // float4 groups per lane and row in flight
  const int groups = K >> 2;
  const float* xr[2];
  const int tt[2] = {t_a, t_b};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int src = 0;
    if (tt[i] >= 0) {
      src = norm.row_index ? norm.row_index[t0 + tt[i]] : t0 + tt[i];
      if (src < 0 || src >= norm.src_rows) {
        if (lane == 0) ls_record_fault(err, LS_DEV_ROW_RANGE, t0 + tt[i]);
        src = 0;
      }
    }
    xr[i] = norm.h + (int64_t)src * K;
  }
  float ss[2] = {0.f, 0.f};
  for (int g0 = lane; g0 < groups; g0 += 32 * U) {
    float4 v[2][U];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int g = g0 + 32 * u;
        v[i][u] = (tt[i] >= 0 && g < groups) ? *reinterpret_cast<const float4*>(xr[i] + 4 * g)
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (g0 + 32 * u < groups) {
          ss[i] = fmaf(v[i][u].x, v[i][u].x, ss[i]); ss[i] = fmaf(v[i][u].y, v[i][u].y, ss[i]);
          ss[i] = fmaf(v[i][u].z, v[i][u].z, ss[i]); ss[i] = fmaf(v[i][u].w, v[i][u].w, ss[i]);
        }
      }
  }
  float rstd[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) rstd[i] = 1.0f / sqrtf(ls_warp_sum(ss[i]) / (float)K + norm.eps);
  int j = 0;
  for (int g = (k_lo >> 2) + lane; g < (k_hi >> 2); g += 32, ++j) {
    float4 v[2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
      v[i] = tt[i] >= 0 ? *reinterpret_cast<const float4*>(xr[i] + 4 * g) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 gn;
    if (j < GAIN_KEEP) {
      gn = gain_kept[0];
#pragma unroll
      for (int q = 1; q < GAIN_KEEP; ++q)
        if (j == q) gn = gain_kept[q];
    } else {
      gn = load_gain4(norm, g);
    }
    const int k = 4 * g - k_lo;                      // column within the share
    const int kb = k >> 6, kk = k & 63;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (tt[i] < 0) continue;
      const int t = tt[i];
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[i].x * rstd[i] * gn.x, v[i].y * rstd[i] * gn.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(v[i].z * rstd[i] * gn.z, v[i].w * rstd[i] * gn.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(x_region + t * 128 + kb * (BN * 128) + (((kk >> 3) ^ (t & 7)) << 4) + (kk & 7) * 2) =
          packed;
    }
  }
  // columns of the last k-block past K: the weight's are zero there, these must not be NaN
  for (int k = k_hi - k_lo + 4 * lane; k < num_kb * BK; k += 128) {
    const int kb = k >> 6, kk = k & 63;
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (tt[i] >= 0)
        *reinterpret_cast<uint2*>(x_region + tt[i] * 128 + kb * (BN * 128) + (((kk >> 3) ^ (tt[i] & 7)) << 4) +
                                  (kk & 7) * 2) = make_uint2(0u, 0u);
  }
}

template <int BN, int EPI, typename TC, bool NORM>
__global__ void __launch_bounds__(192, 1)
gemm_tc_few_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const NormArgs norm, const LsQkvStore heads, TC* __restrict__ C, int T, int N, int K,
                   int64_t ldc, int kb_per_share, int shares, const FewLayout lay, int* err) {
  constexpr int A_TILES = EPI == 2 ? 2 : 1;
  constexpr int STAGE_BYTES = A_TILES * A_BYTES + (NORM ? 0 : BN * BK * 2);
  constexpr int REGION_COLS = A_TILES * BN;
  constexpr uint32_t ACC_COLS = (uint32_t)tmem_cols(REGION_COLS);
  ls_dependency_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t x_base = base + lay.x_off;
  float* recv = reinterpret_cast<float*>(aligned + lay.recv_off);
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + lay.bars_off);
  uint64_t* full = bars;                          // [stages] operands landed
  uint64_t* empty = bars + MAX_STAGES;            // [stages] MMAs have read the stage
  uint64_t* acc_full = bars + 2 * MAX_STAGES;     // the accumulator is complete
  uint64_t* x_ready = acc_full + 1;               // NORM: the token operand is in shared memory
  uint64_t* recv_bar = acc_full + 2;              // every share's columns for this block have arrived
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 3);
  volatile uint32_t* failed = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = lay.stages;
  const int rank = (int)blockIdx.z;               // the cluster is the z extent of the grid
  const int n0 = blockIdx.x * BM;
  const int t0 = blockIdx.y * BN;
  const int total_kb = (K + BK - 1) / BK;
  const int kb_begin = rank * kb_per_share;
  int kb_end = kb_begin + kb_per_share;
  if (kb_end > total_kb) kb_end = total_kb;
  const int num_kb = kb_end - kb_begin;
  const int valid = T - t0 < BN ? T - t0 : BN;    // token columns of this tile
  const int my_cols = valid > rank ? (valid - rank + shares - 1) / shares : 0;   // columns rank, rank + shares, ...

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(x_ready, 4);
    mbar_init(recv_bar, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // every share sends A_TILES x 128 floats for each column this block folds
    if (my_cols > 0) mbar_expect_tx(recv_bar, (uint32_t)(my_cols * shares * A_TILES * BM * 4));
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    if (!NORM) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(ACC_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  cluster_arrive();                               // this block's barriers exist; waited for before the first push
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // The weights do not depend on the previous kernel; the token operand read by TMA does:
    // the first round of the ring takes its weights before the wait and its tokens after.
    // A stage of the first round is a lane's: a thread gets one TMA instruction out about
    // every 300 ns, so the lanes issue side by side what one lane would issue in a row.
    const int first_round = num_kb < stages ? num_kb : stages;
    if (lane < first_round) {
      const uint32_t stage = base + (uint32_t)lane * STAGE_BYTES;
      mbar_expect_tx(&full[lane], STAGE_BYTES);
      const int kx = (kb_begin + lane) * BK;
      tma_load_2d(stage, &map_w, kx, n0, &full[lane]);
      if (EPI == 2) tma_load_2d(stage + A_BYTES, &map_w, kx, N + n0, &full[lane]);
    }
    if (!NORM) {
      ls_dependency_wait();
      if (lane < first_round)
        tma_load_2d(base + (uint32_t)lane * STAGE_BYTES + A_TILES * A_BYTES, &map_x, (kb_begin + lane) * BK, t0,
                    &full[lane]);
    }
    __syncwarp();
    if (lane == 0) {
      int issued = first_round;
      int s = 0;                                  // kb % stages and the parity of kb / stages, without dividing
      uint32_t phase = 1u;
      for (int kb = first_round; kb < num_kb; ++kb) {
        if (*failed || !mbar_wait(&empty[s], phase ^ 1u)) {
          *failed = 1;
          ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 400 + s);
          break;
        }
        const uint32_t stage = base + (uint32_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        const int kx = (kb_begin + kb) * BK;
        tma_load_2d(stage, &map_w, kx, n0, &full[s]);
        if (EPI == 2) tma_load_2d(stage + A_BYTES, &map_w, kx, N + n0, &full[s]);
        if (!NORM) tma_load_2d(stage + A_TILES * A_BYTES, &map_x, kx, t0, &full[s]);
        issued = kb + 1;
        if (++s == stages) {
          s = 0;
          phase ^= 1u;
        }
      }
      if (*failed) {
        // wait (bounded) for the copies still in flight before the block exits
        const int first = issued > stages ? issued - stages : 0;
        for (int kb = first; kb < issued; ++kb) mbar_wait(&full[kb % stages], (uint32_t)(kb / stages) & 1u);   // cold path
      }
    }
    __syncwarp();
    cluster_wait();
  } else if (warp == 1) {
    // the whole warp walks the loop and one elected lane issues (see gemm_tc_cluster_kernel)
    constexpr uint32_t idesc = instr_desc(BM, BN);
    const bool issuer = elect_one();
    bool ok = true;
    if (NORM) {
      ok = __all_sync(0xffffffffu, mbar_wait(x_ready, 0));
      if (!ok) {
        *failed = 1;
        if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 560);
      }
    }
    int s = 0;
    uint32_t phase = 0u;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      ok = __all_sync(0xffffffffu, mbar_wait(&full[s], phase));     // runs out too when the producer gave up
      if (!ok) {
        *failed = 1;
        if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 500 + s);
        break;
      }
      fence_after_sync();
      const uint32_t stage = base + (uint32_t)s * STAGE_BYTES;
      const uint32_t xs = NORM ? x_base + (uint32_t)(kb * BN * 128) : stage + A_TILES * A_BYTES;
      // a step of 16 elements along K is 32 bytes: 2 in the descriptor's address field
      const uint64_t adesc = desc_k_major(stage), udesc = desc_k_major(stage + A_BYTES), bdesc = desc_k_major(xs);
      if (issuer) {
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
          umma(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, acc);
          if (EPI == 2) umma(tmem_base + BN, udesc + 2 * k, bdesc + 2 * k, idesc, acc);
        }
        if (kb + stages < num_kb) umma_commit(&empty[s]);     // only a stage that is filled again
      }
      __syncwarp();
      if (++s == stages) {
        s = 0;
        phase ^= 1u;
      }
    }
    if (ok && issuer) umma_commit(acc_full);
    __syncwarp();
    cluster_wait();
  } else {
    // epilogue warps: warp w may touch tensor-memory lanes 32*(w%4) .. +32
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int n = n0 + row;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int k_lo = kb_begin * BK;
    const int k_hi = kb_end * BK < K ? kb_end * BK : K;
    float4 gain_kept[GAIN_KEEP];
    if (NORM) {
#pragma unroll
      for (int j = 0; j < GAIN_KEEP; ++j) {
        const int g = (k_lo >> 2) + lane + 32 * j;
        gain_kept[j] = g < (k_hi >> 2) ? load_gain4(norm, g) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    // q/k/v epilogue: where this warp's first head goes depends on the step's inputs alone
    LsHeadTarget first_target;
    if constexpr (EPI == 3) {
      if (quad < my_cols * (BM / heads.d)) {
        const int per_tile = BM / heads.d;
        const int slot = quad / per_tile, j = quad - slot * per_tile;
        const int head = n0 / heads.d + j;
        if (head < heads.nq + 2 * heads.nkv)
          first_target = ls_qkv_head_target(heads, t0 + rank + slot * shares, head, 2, lane, err);
        else
          first_target.dst = nullptr;
      }
    }
    ls_dependency_wait();
    float first_old = 0.f;      // residual epilogue: the old value of the first column this block folds
    if (EPI == 1 && rank < valid && n < N) first_old = ls_to_float<TC>(C[(int64_t)(t0 + rank) * ldc + n]);
    if (NORM) {
      for (int t = warp - 2; t < valid; t += 8)
        normed_rows_to_smem<BN>(norm, gain_kept, aligned + lay.x_off, t, t + 4 < valid ? t + 4 : -1, t0, K, k_lo, k_hi,
                                num_kb, lane, err);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(x_ready);
    }
    cluster_wait();             // every block of the cluster has its barriers and may be written to
    bool ok = mbar_wait(acc_full, 0);
    if (!ok) {
      *failed = 1;
      if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 600 + quad);
    }
    ok = __all_sync(0xffffffffu, ok);
    fence_after_sync();
    const uint32_t recv_mine = smem_u32(recv) + (uint32_t)(rank * lay.slots * A_TILES * BM + row) * 4u;
    const uint32_t recv_bar_addr = smem_u32(recv_bar);
    if (ok) {
      // column c of the tile goes to the block of rank c % shares, into its slot c / shares
#pragma unroll
      for (int part = 0; part < A_TILES; ++part) {
        int dest = 0, slot = 0;
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t g[16];
          tmem_ld16(lane_base + part * BN + c0, g);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < valid)
              st_async_f32(map_to_rank(recv_mine + (uint32_t)((slot * A_TILES + part) * BM) * 4u, dest),
                           __uint_as_float(g[j]), map_to_rank(recv_bar_addr, dest));
            if (++dest == shares) {
              dest = 0;
              ++slot;
            }
          }
        }
      }
    }
    // a block that failed pushes nothing: its peers' waits run out and they record it too
    bool got = true;
    if (my_cols > 0) {
      got = mbar_wait_long(recv_bar, 0);
      if (!got) {
        *failed = 1;
        if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 700 + quad);
      }
    }
    if constexpr (EPI == 3) {
      // the folded columns, rounded as a stored projection would be, then a warp per head
      __nv_bfloat16* folded = reinterpret_cast<__nv_bfloat16*>(aligned + lay.head_off);
      const bool fold_ok = got && !*failed;
      if (fold_ok) {
        for (int slot = 0; slot < my_cols; ++slot) {
          const float* p = recv + slot * BM + row;
          const int share_stride = lay.slots * BM;
          float vg[MAX_SHARES];
#pragma unroll
          for (int r = 0; r < MAX_SHARES; ++r) vg[r] = r < shares ? p[r * share_stride] : 0.f;
          float g = 0.f;
#pragma unroll
          for (int r = 0; r < MAX_SHARES; ++r)
            if (r < shares) g += vg[r];
          folded[slot * BM + row] = __float2bfloat16_rn(g);
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");      // the four epilogue warps
      if (fold_ok) {
        const int per_tile = BM / heads.d;                 // heads of this tile of rows
        for (int job = quad; job < my_cols * per_tile; job += 4) {
          const int slot = job / per_tile, j = job - slot * per_tile;
          const int head = n0 / heads.d + j;
          if (head >= heads.nq + 2 * heads.nkv) continue;
          const LsHeadTarget target =
              job == quad ? first_target
                          : ls_qkv_head_target(heads, t0 + rank + slot * shares, head, 2, lane, err);
          ls_qkv_head_write<__nv_bfloat16>(heads, folded + slot * BM + j * heads.d, target, lane);
        }
      }
    } else if (got && !*failed && n < N) {
      for (int slot = 0; slot < lay.slots; ++slot) {
        const int c = rank + slot * shares;
        if (c >= valid) break;
        const float* p = recv + (slot * A_TILES) * BM + row;
        const int share_stride = lay.slots * A_TILES * BM;
        float vg[MAX_SHARES], vu[MAX_SHARES];
#pragma unroll
        for (int r = 0; r < MAX_SHARES; ++r) {
          vg[r] = r < shares ? p[r * share_stride] : 0.f;
          if (EPI == 2) vu[r] = r < shares ? p[r * share_stride + BM] : 0.f;
        }
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int r = 0; r < MAX_SHARES; ++r) {
          if (r < shares) {
            g += vg[r];
            if (EPI == 2) u += vu[r];
          }
        }
        TC* cp = C + (int64_t)(t0 + c) * ldc + n;
        if (EPI == 1) {
          const float before = slot == 0 ? first_old : ls_to_float<TC>(*cp);
          *cp = ls_from_float<TC>(before + g);
        } else {
          epilogue_store<EPI, TC>(cp, g, u);
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// The persistent form: a block per SM walks output tiles, and within a tile the
// shares of K, in one stream.  Two accumulator regions in tensor memory
// alternate share by share: while the MMA warp fills one, the epilogue warps
// drain the other into the running sum they keep in registers
// (((0 + p_0) + p_1) + ...), and after a tile's last share they write it out,
// all while the next tile's products already run.
// ---------------------------------------------------------------------------
// EW epilogue warps: 4 (192 threads; up to 128 running sums per thread) or 8 (320 threads: the
// silu-mul epilogue at 128 tokens has 256 columns, which two groups of four warps split).
template <int BN, int EPI, typename TC, int EW>
__global__ void __launch_bounds__(EW == 8 ? 320 : 192, 1)
gemm_tc_walk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    TC* __restrict__ C, int T, int N, int K, int64_t ldc, int kb_per_share, int shares,
                    int tiles_n, int tiles_total, int* err) {
  using S = Shape<BN, EPI>;
  constexpr int COLS = S::REGION_COLS;           // columns of one accumulator region
  constexpr int GROUPS = EW / 4;                 // epilogue warpgroups: each takes BN / GROUPS tokens
  constexpr int TOK = BN / GROUPS;               // tokens per epilogue thread
  constexpr int SUMS = S::A_TILES * TOK;         // running sums per epilogue thread
  constexpr int EPI_FIRST = 2;                   // first epilogue warp
  static_assert(SUMS <= 128 && TOK % 16 == 0 && 2 * COLS <= 512, "token tile too wide for register sums");
  ls_dependency_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + (size_t)S::STAGES * S::STAGE_BYTES);
  uint64_t* full = bars;                        // [STAGES]
  uint64_t* empty = bars + S::STAGES;           // [STAGES]
  uint64_t* acc_full = bars + 2 * S::STAGES;    // [2] a share's accumulator is complete
  uint64_t* acc_empty = acc_full + 2;           // [2] the epilogue has drained it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* failed = tmem_slot + 1;
  constexpr uint32_t ACC_COLS = (uint32_t)tmem_cols(2 * COLS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int r = 0; r < 2; ++r) {
      mbar_init(&acc_full[r], 1);
      mbar_init(&acc_empty[r], EW);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(ACC_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  ls_dependency_wait();

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;                                 // k-blocks issued so far, over all tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles_total && ok; tile += gridDim.x) {
        const int n0 = (tile % tiles_n) * BM, t0 = (tile / tiles_n) * BN;
        for (int kb = 0; kb < total_kb; ++kb, ++it) {
          const int s = it % S::STAGES;
          const uint32_t phase = (uint32_t)(it / S::STAGES) & 1u;
          if (*failed || !mbar_wait(&empty[s], phase ^ 1u)) {
            *failed = 1;
            ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 100 + s);
            ok = false;
            break;
          }
          const uint32_t stage = base + (uint32_t)s * S::STAGE_BYTES;
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          tma_load_2d(stage, &map_w, kb * BK, n0, &full[s]);
          if (EPI == 2) tma_load_2d(stage + A_BYTES, &map_w, kb * BK, N + n0, &full[s]);
          tma_load_2d(stage + S::A_TILES * A_BYTES, &map_x, kb * BK, t0, &full[s]);
        }
      }
      if (!ok) {
        // wait (bounded) for the copies still in flight before the block exits
        const int first = it > S::STAGES ? it - S::STAGES : 0;
        for (int j = first; j < it; ++j) mbar_wait(&full[j % S::STAGES], (uint32_t)(j / S::STAGES) & 1u);
      }
    }
  } else if (warp == 1) {
    // the whole warp walks the loop and one elected lane issues (see gemm_tc_cluster_kernel)
    constexpr uint32_t idesc = instr_desc(BM, BN);
    const bool issuer = elect_one();
    int s = 0, sc = 0;                            // the stage in turn; shares consumed so far
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles_total && ok; tile += gridDim.x) {
      for (int r = 0; r < shares && ok; ++r, ++sc) {
        const int region = sc & 1;
        const uint32_t acc_addr = tmem_base + (uint32_t)(region * COLS);
        ok = __all_sync(0xffffffffu, !*failed && mbar_wait(&acc_empty[region], ((uint32_t)(sc >> 1) & 1u) ^ 1u));
        if (!ok) {
          *failed = 1;
          if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 250 + region);
          break;
        }
        fence_after_sync();
        const int kb_lo = r * kb_per_share;
        int kb_hi = kb_lo + kb_per_share;
        if (kb_hi > total_kb) kb_hi = total_kb;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          ok = __all_sync(0xffffffffu, !*failed && mbar_wait(&full[s], phase));
          if (!ok) {
            *failed = 1;
            if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 200 + s);
            break;
          }
          fence_after_sync();
          const uint32_t stage = base + (uint32_t)s * S::STAGE_BYTES;
          const uint64_t adesc = desc_k_major(stage), udesc = desc_k_major(stage + A_BYTES);
          const uint64_t bdesc = desc_k_major(stage + S::A_TILES * A_BYTES);
          if (issuer) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint32_t acc = (kb == kb_lo && k == 0) ? 0u : 1u;
              umma(acc_addr, adesc + 2 * k, bdesc + 2 * k, idesc, acc);
              if (EPI == 2) umma(acc_addr + BN, udesc + 2 * k, bdesc + 2 * k, idesc, acc);
            }
            umma_commit(&empty[s]);
          }
          __syncwarp();
          if (++s == S::STAGES) {
            s = 0;
            phase ^= 1u;
          }
        }
        if (ok && issuer) umma_commit(&acc_full[region]);
        __syncwarp();
      }
    }
  } else if (warp >= EPI_FIRST) {
    // epilogue: warp w may touch tensor-memory lanes 32*(w%4) .. +32
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int tok_first = ((warp - EPI_FIRST) >> 2) * TOK;      // this warpgroup's tokens of the tile
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    float sum[SUMS];
    int sc = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles_total && ok; tile += gridDim.x) {
      const int n = (tile % tiles_n) * BM + row, t0 = (tile / tiles_n) * BN;
      for (int r = 0; r < shares; ++r, ++sc) {
        const int region = sc & 1;
        bool got = mbar_wait(&acc_full[region], (uint32_t)(sc >> 1) & 1u);
        if (!got) {
          *failed = 1;
          if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 350 + quad);
        }
        ok = __all_sync(0xffffffffu, got);
        if (!ok) break;
        fence_after_sync();
#pragma unroll
        for (int part = 0; part < S::A_TILES; ++part) {          // gate, then (silu-mul) up
#pragma unroll
          for (int c0 = 0; c0 < TOK; c0 += 32) {
            uint32_t g[32];
            const uint32_t col = (uint32_t)(region * COLS + part * BN + tok_first + c0);
            if (TOK - c0 >= 32) {
              tmem_ld32(lane_base + col, g);
            } else {
              tmem_ld16(lane_base + col, g);
            }
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < TOK)
                sum[part * TOK + c0 + j] = (r == 0 ? 0.f : sum[part * TOK + c0 + j]) + __uint_as_float(g[j]);
          }
        }
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[region]);
      }
      if (ok && n < N) {
#pragma unroll
        for (int c0 = 0; c0 < TOK; c0 += 8) {
          const int tb = t0 + tok_first + c0;
          if (tb < T) {
            float old[8];
            if (EPI == 1) {
              // the residual rows are fetched together before any is written back
#pragma unroll
              for (int j = 0; j < 8; ++j)
                old[j] = (tb + j < T) ? ls_to_float<TC>(C[(int64_t)(tb + j) * ldc + n]) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int t = tb + j;
              if (t < T) {
                TC* c = C + (int64_t)t * ldc + n;
                const float a = sum[c0 + j];
                if (EPI == 0) *c = ls_from_float<TC>(a);
                else if (EPI == 1) *c = ls_from_float<TC>(old[j] + a);
                else *c = ls_from_float<TC>(silu_mul(a, sum[TOK + c0 + j]));
              }
            }
          }
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Many tokens (more than 128): the persistent kernel with the tokens on the MMA's M side.
// A tile is 128 tokens x FN features (256, or 128 for silu-mul whose weight tile is 128 gate
// rows and the 128 up rows of the same features: one MMA of N = 256 makes both).  A token is
// a lane of tensor memory and a thread of the epilogue, whose outputs for that token lie side
// by side in memory and leave in 16-byte pieces (with the weights on the M side a thread had
// one feature of 128 tokens and wrote 128 scattered elements, a quarter of the kernel's
// time).  An output element is the same dot product in the same order of k as in the other
// kernels, shares and all; the eight epilogue warps are two groups that split the features.
// ---------------------------------------------------------------------------
// FN: features per tile: 256, or 128 where 256 would leave SMs without a tile (and always 128
// for silu-mul, whose stage holds 128 gate rows and 128 up rows).
// CTAS: 1, or 2 for a pair of blocks (a cluster) on one tile of 256 tokens: each block holds its
// own 128 tokens and half of the weight rows, one thread of the first block issues MMAs of
// M = 256 (tcgen05 cta_group::2) that read both blocks' shared memory and write each block's
// 128 tokens into its own tensor memory.  A block then loads 2/3 (3/4 at FN = 128) of the
// bytes per MMA cycle, and what bounds this kernel is what L2 delivers.
template <int EPI, int FN, int CTAS>
struct RowsShape {
  static_assert(FN == 128 || (FN == 256 && EPI != 2), "tile widths");
  static_assert(CTAS == 1 || CTAS == 2, "a block or a pair");
  static constexpr int W_ROWS = EPI == 2 ? 256 : FN;        // weight rows per k-block (MMA N)
  static constexpr int W_BOXES = (EPI == 2 && CTAS == 1) ? 2 : 1;   // gate and up rows of one block come apart
  static constexpr int X_BYTES = BM * BK * 2;               // 128 tokens
  static constexpr int W_BYTES = W_ROWS / CTAS * BK * 2;    // this block's part of the weight rows
  static constexpr int KB_BYTES = X_BYTES + W_BYTES;        // a k-block: 48, 32 or 24 KB
  static constexpr int STAGE_KB = 2;                        // k-blocks per stage: one wait and one commit for both
  static constexpr int STAGE_BYTES = STAGE_KB * KB_BYTES;
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;
  static constexpr int BOXES = STAGE_KB * (1 + W_BOXES);    // TMA loads per stage, a lane each
  static constexpr int STAGING = 8 * 4096;                  // a warp's 32 tokens x 128 bytes on their way out
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + STAGING + 1024 + 256;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// a TMA load whose bytes count on a barrier of the pair's first block
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
template <int CTAS>
__device__ __forceinline__ void tma_load_2d_any(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  if constexpr (CTAS == 2) {
    tma_load_2d_pair(dst, map, x, y, bar);
  } else {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
  }
}
__device__ __forceinline__ void umma_pair(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the barrier at this offset in both blocks of the pair gets an arrival when the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  // (not .release.cluster: that waits for the thread's earlier accesses to be seen by the whole
  // cluster, 250 ns and more an arrival; the tensor-memory reads this orders are complete already)
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

template <int EPI, int FN, int CTAS, typename TC>
__global__ void __launch_bounds__(320, 1)
gemm_tc_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_c, int store_by_tma, TC* __restrict__ C, int T, int N,
                    int K, int64_t ldc, int kb_per_share, int shares, int tiles_t, int tiles_total, int* err) {
  using S = RowsShape<EPI, FN, CTAS>;
  constexpr int COLS = 256;                      // columns of one accumulator region
  constexpr int OUT = FN / 2;                    // outputs per epilogue thread (features of its group)
  constexpr int SUMS = S::W_ROWS / 2;            // running sums per epilogue thread
  ls_dependency_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint8_t* staging = aligned + (size_t)S::STAGES * S::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + S::STAGING);
  uint64_t* full = bars;                        // [STAGES] (a pair uses those of its first block)
  uint64_t* empty = bars + S::STAGES;           // [STAGES]
  uint64_t* acc_full = bars + 2 * S::STAGES;    // [2] a share's accumulator is complete
  uint64_t* acc_empty = acc_full + 2;           // [2] the epilogue has drained it (a pair: the first block's)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* failed = tmem_slot + 1;
  constexpr uint32_t ACC_COLS = 512;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (K + BK - 1) / BK;
  const int rank = CTAS == 2 ? (int)cluster_rank() : 0;     // this block's place in its pair
  const int first_tile = blockIdx.x / CTAS, tile_step = gridDim.x / CTAS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int r = 0; r < 2; ++r) {
      mbar_init(&acc_full[r], 1);
      mbar_init(&acc_empty[r], 8 * CTAS);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    if constexpr (CTAS == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(ACC_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(ACC_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  fence_before_sync();
  __syncthreads();
  if constexpr (CTAS == 2) {        // the peer's barriers exist before anything arrives on them
    cluster_arrive();
    cluster_wait();
  }
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  ls_dependency_wait();

  // tiles are walked token-tile fastest: the blocks running at one time share a few weight tiles
  if (warp == 0) {
    // A stage is up to two k-blocks of one share; each of its boxes goes out from a lane of its
    // own (a thread gets a TMA load out only every few hundred cycles, lanes side by side scale).
    if (lane < S::BOXES) {
      const int half = lane / (1 + S::W_BOXES), part = lane % (1 + S::W_BOXES);   // k-block of the stage; tokens, weights
      const uint32_t full0 = CTAS == 2 ? map_to_rank(smem_u32(&full[0]), 0) : smem_u32(&full[0]);
      int s = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < tiles_total && ok; tile += tile_step) {
        const int t0 = (tile % tiles_t) * (BM * CTAS) + rank * BM, n0 = (tile / tiles_t) * FN;
        // this block's weight rows: all of the tile's; of a pair, the gate rows in the first block
        // and the up rows in the second, or each its half of the features
        const int w0 = EPI == 2 ? (CTAS == 2 ? rank * N + n0 : n0 + (part == 2 ? N : 0)) : n0 + rank * (FN / CTAS);
        const CUtensorMap* map = part == 0 ? &map_x : &map_w;
        const int y = part == 0 ? t0 : w0;
        const uint32_t within = (uint32_t)(half * S::KB_BYTES + (part == 0 ? 0 : S::X_BYTES + (part - 1) * (S::W_BYTES / 2)));
        for (int r = 0; r < shares && ok; ++r) {
          const int kb_lo = r * kb_per_share;
          int kb_hi = kb_lo + kb_per_share;
          if (kb_hi > total_kb) kb_hi = total_kb;
          for (int kb = kb_lo; kb < kb_hi; kb += S::STAGE_KB) {
            const int n = kb_hi - kb < S::STAGE_KB ? kb_hi - kb : S::STAGE_KB;
            if (*failed || !mbar_wait(&empty[s], phase ^ 1u)) {
              *failed = 1;
              if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 900 + s);
              ok = false;
              break;
            }
            if (lane == 0 && rank == 0) mbar_expect_tx(&full[s], (uint32_t)(CTAS * n * S::KB_BYTES));
            if (half < n)
              tma_load_2d_any<CTAS>(base + (uint32_t)s * S::STAGE_BYTES + within, map, (kb + half) * BK, y,
                                    full0 + (uint32_t)s * 8u);
            ++issued;
            if (++s == S::STAGES) {
              s = 0;
              phase ^= 1u;
            }
          }
        }
      }
      if (!ok && lane == 0 && rank == 0) {
        // wait (bounded) for the copies still in flight before the block exits
        for (int j = issued > S::STAGES ? issued - S::STAGES : 0; j < issued; ++j)
          mbar_wait(&full[j % S::STAGES], (uint32_t)(j / S::STAGES) & 1u);
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop and one elected lane issues: what the instructions take
    // (descriptors, addresses) is then the same in every lane and stays in uniform registers;
    // inside a branch of one lane each MMA paid for moving them there.
    if (rank == 0) {
      constexpr uint32_t idesc = instr_desc(BM * CTAS, S::W_ROWS);
      const bool issuer = elect_one();
      int s = 0, sc = 0;                          // the stage in turn; shares consumed so far
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < tiles_total && ok; tile += tile_step) {
        for (int r = 0; r < shares && ok; ++r, ++sc) {
          const int region = sc & 1;
          const uint32_t acc_addr = tmem_base + (uint32_t)(region * COLS);
          ok = __all_sync(0xffffffffu, !*failed && mbar_wait(&acc_empty[region], ((uint32_t)(sc >> 1) & 1u) ^ 1u));
          if (!ok) {
            *failed = 1;
            if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 950 + region);
            break;
          }
          fence_after_sync();
          const int kb_lo = r * kb_per_share;
          int kb_hi = kb_lo + kb_per_share;
          if (kb_hi > total_kb) kb_hi = total_kb;
          for (int kb = kb_lo; kb < kb_hi; kb += S::STAGE_KB) {
            const int n = kb_hi - kb < S::STAGE_KB ? kb_hi - kb : S::STAGE_KB;
            ok = __all_sync(0xffffffffu, mbar_wait(&full[s], phase));
            if (!ok) {
              *failed = 1;
              if (issuer) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 920 + s);
              break;
            }
            fence_after_sync();
            const uint32_t stage = base + (uint32_t)s * S::STAGE_BYTES;
            const uint64_t adesc = desc_k_major(stage), bdesc = desc_k_major(stage + S::X_BYTES);
            if (issuer) {
#pragma unroll
              for (int h = 0; h < S::STAGE_KB; ++h) {
                if (h < n) {
#pragma unroll
                  for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint32_t acc = (kb == kb_lo && h == 0 && k == 0) ? 0u : 1u;
                    const uint64_t step = (uint64_t)((h * S::KB_BYTES) >> 4) + 2 * k;
                    if constexpr (CTAS == 2) umma_pair(acc_addr, adesc + step, bdesc + step, idesc, acc);
                    else umma(acc_addr, adesc + step, bdesc + step, idesc, acc);
                  }
                }
              }
              if constexpr (CTAS == 2) umma_commit_pair(&empty[s]);
              else umma_commit(&empty[s]);
            }
            __syncwarp();
            if (++s == S::STAGES) {
              s = 0;
              phase ^= 1u;
            }
          }
          if (ok && issuer) {
            if constexpr (CTAS == 2) umma_commit_pair(&acc_full[region]);
            else umma_commit(&acc_full[region]);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // epilogue: warp w may touch tensor-memory lanes 32*(w%4) .. +32; this thread has token `row`
    // of the block's 128 and the features OUT * group .. + OUT of it (for silu-mul their gate and up sums)
    const int quad = warp & 3;
    const int group = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    float sum[SUMS];
    int sc = 0;
    bool ok = true;
    for (int tile = first_tile; tile < tiles_total && ok; tile += tile_step) {
      const int t = (tile % tiles_t) * (BM * CTAS) + rank * BM + row, n_first = (tile / tiles_t) * FN + group * OUT;
      for (int r = 0; r < shares; ++r, ++sc) {
        const int region = sc & 1;
        bool got = mbar_wait(&acc_full[region], (uint32_t)(sc >> 1) & 1u);
        if (!got) {
          *failed = 1;
          if (lane == 0) ls_record_fault(err, LS_DEV_WAIT_TIMEOUT, 970 + quad);
        }
        ok = __all_sync(0xffffffffu, got);
        if (!ok) break;
        fence_after_sync();
        // columns of the region: store/residual: this group's 128 features; silu-mul: gate columns
        // OUT * group .. and up columns 128 + OUT * group ..
#pragma unroll
        for (int c0 = 0; c0 < SUMS; c0 += 32) {
          uint32_t g[32];
          const int col = EPI == 2 ? (c0 < OUT ? group * OUT + c0 : 128 + group * OUT + (c0 - OUT)) : group * OUT + c0;
          tmem_ld32(lane_base + (uint32_t)(region * COLS + col), g);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[c0 + j] = (r == 0 ? 0.f : sum[c0 + j]) + __uint_as_float(g[j]);
        }
        fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTAS == 2) mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty[region]), 0));
          else mbar_arrive(&acc_empty[region]);
        }
      }
      if (!ok) break;
      constexpr int PER = 16 / (int)sizeof(TC);                // outputs of a 16-byte piece
      constexpr int CH = 8 * PER;                              // outputs of a 128-byte chunk of a row
      // whole 16-byte pieces of rows that start on 16-byte boundaries (the same answer in every lane)
      const bool pieces = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc % PER) == 0 && n_first + OUT <= N;
      if (pieces) {
        // Through shared memory, 128 bytes of each of the warp's 32 tokens at a time: a lane puts
        // its token's chunk there, then eight lanes together take one token's chunk to memory, four
        // tokens an instruction.  (A lane writing its own token's pieces touched 32 lines per
        // instruction, and the tile's stores took as long as its MMAs.)
        uint8_t* mine = staging + (warp - 2) * 4096;
        const int t_warp = t - lane;                           // the warp's first token
        TC* cbase = C + (int64_t)t_warp * ldc + n_first;
#pragma unroll
        for (int c0 = 0; c0 < OUT; c0 += CH) {
          if (EPI != 1 && store_by_tma) {                      // the store before has read the staging chunk
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float v[PER];
#pragma unroll
            for (int e = 0; e < PER; ++e) {
              const float a = sum[c0 + j * PER + e];
              v[e] = EPI == 2 ? silu_mul(a, sum[OUT + c0 + j * PER + e]) : a;
            }
            uint4 piece;
            if constexpr (sizeof(TC) == 4) {
              piece = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
            } else {
              piece.x = pack_bf16(v[0], v[1]); piece.y = pack_bf16(v[2], v[3]);
              piece.z = pack_bf16(v[4], v[5]); piece.w = pack_bf16(v[6], v[7]);
            }
            *reinterpret_cast<uint4*>(mine + lane * 128 + ((j ^ (lane & 7)) << 4)) = piece;
          }
          __syncwarp();
          const int slot = lane & 7;
          if constexpr (EPI == 1) {
            constexpr int AT_ONCE = SUMS > 64 ? 4 : 8;         // old values asked for together (registers allowing)
#pragma unroll
            for (int i0 = 0; i0 < 8; i0 += AT_ONCE) {
              float4 old[AT_ONCE];
#pragma unroll
              for (int i = 0; i < AT_ONCE; ++i) {
                const int r = (i0 + i) * 4 + (lane >> 3);
                if (t_warp + r < T) old[i] = *reinterpret_cast<const float4*>(cbase + (int64_t)r * ldc + c0 + slot * PER);
              }
#pragma unroll
              for (int i = 0; i < AT_ONCE; ++i) {
                const int r = (i0 + i) * 4 + (lane >> 3);
                const float4 add = *reinterpret_cast<const float4*>(mine + r * 128 + ((slot ^ (r & 7)) << 4));
                if (t_warp + r < T)
                  *reinterpret_cast<float4*>(cbase + (int64_t)r * ldc + c0 + slot * PER) =
                      make_float4(add.x + old[i].x, add.y + old[i].y, add.z + old[i].z, add.w + old[i].w);
              }
            }
          } else if (store_by_tma) {
            // the chunk (its layout is the 128-byte swizzle) leaves as one TMA store, which this
            // warp does not wait for: tokens past T and features past N are cut off by the map
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&map_c),
                           "r"(smem_u32(mine)), "r"(n_first + c0), "r"(t_warp)
                           : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + (lane >> 3);
              const uint4 piece = *reinterpret_cast<const uint4*>(mine + r * 128 + ((slot ^ (r & 7)) << 4));
              if (t_warp + r < T) *reinterpret_cast<uint4*>(cbase + (int64_t)r * ldc + c0 + slot * PER) = piece;
            }
          }
          __syncwarp();
        }
      } else if (t < T) {
        TC* crow = C + (int64_t)t * ldc + n_first;
#pragma unroll
        for (int c0 = 0; c0 < OUT; ++c0) {
          if (n_first + c0 < N) {
            const float a = sum[c0];
            const float v = EPI == 2 ? silu_mul(a, sum[OUT + c0]) : a;
            crow[c0] = ls_from_float<TC>(EPI == 1 ? v + ls_to_float<TC>(crow[c0]) : v);
          }
        }
      }
    }
    if (EPI != 1 && store_by_tma && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  if constexpr (CTAS == 2) {        // nothing of the pair's is in flight towards a block that has left
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 2) {
    fence_after_sync();
    if constexpr (CTAS == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_COLS) : "memory");
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
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
  }
  return fn;
}

// rows x K bfloat16, row pitch ld elements; box of box_rows x 64 with 128-byte swizzle
bool make_map(CUtensorMap* map, const void* ptr, int rows, int K, int64_t ld, int box_rows) {
  EncodeTiled enc = encode_fn();
  if (enc == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Plan {
  int shares, kb_per_share, in_cluster, bn;
};

// How a product of T tokens with a weight of N rows and depth K runs.  The shares
// of K depend on the weight alone; T only decides where they run and how wide
// the token tile is, neither of which changes a sum.
Plan make_plan(int T, int N, int K, int epilogue) {
  Plan p;
  const int total_kb = (K + BK - 1) / BK;
  const int want = ls_gemm_tc_k_shares(N, K);
  p.kb_per_share = (total_kb + want - 1) / want;
  p.shares = (total_kb + p.kb_per_share - 1) / p.kb_per_share;    // every share has work
  p.in_cluster = p.shares > 1 && T <= 128;
  p.bn = 16;                                        // token tile of the kernels with the weights on the M side
  while (p.bn < T && p.bn < 128) p.bn *= 2;         // (more than 128 tokens go to the kernel with tokens as rows)
  return p;
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

template <int BN, int EPI, typename TC>
int launch_cluster(const CUtensorMap& mw, const CUtensorMap& mx, void* C, int T, int N,
                   int K, int64_t ldc, const Plan& plan, int* err, cudaStream_t stream) {
  using S = ClusterShape<BN, EPI>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_cluster_kernel<BN, EPI, TC>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM) != cudaSuccess)
      return LS_E_SMEM;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((N + BM - 1) / BM, (T + BN - 1) / BN, plan.shares);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = S::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = plan.shares;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ls_dependent_launch ? 2 : 1;
  LS_COUNT(LS_K_GEMM_TC_CLUSTER);
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_cluster_kernel<BN, EPI, TC>, mw, mx, (TC*)C, T,
                                     N, K, ldc, plan.kb_per_share, plan.shares, err);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

constexpr int MAX_DYNAMIC_SMEM = 227 * 1024;

template <int BN, int EPI, typename TC, bool NORM>
int launch_few(const CUtensorMap& mw, const CUtensorMap& mx, const NormArgs& norm, const LsQkvStore& heads, void* C,
               int T, int N, int K, int64_t ldc, const Plan& plan, int* err, cudaStream_t stream) {
  constexpr int A_TILES = EPI == 2 ? 2 : 1;
  constexpr int STAGE_BYTES = A_TILES * A_BYTES + (NORM ? 0 : BN * BK * 2);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_few_kernel<BN, EPI, TC, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             MAX_DYNAMIC_SMEM) != cudaSuccess)
      return LS_E_SMEM;
    configured = true;
  }
  FewLayout lay;
  lay.slots = (BN + plan.shares - 1) / plan.shares;
  const int x_bytes = NORM ? plan.kb_per_share * BN * 128 : 0;
  const int recv_bytes = plan.shares * lay.slots * A_TILES * BM * 4;
  const int head_bytes = EPI == 3 ? lay.slots * BM * 2 : 0;
  const int bars_bytes = 256;
  const int fit = (MAX_DYNAMIC_SMEM - 1024 - bars_bytes - x_bytes - recv_bytes - head_bytes) / STAGE_BYTES;
  lay.stages = plan.kb_per_share < MAX_STAGES ? plan.kb_per_share : MAX_STAGES;
  if (lay.stages > fit) lay.stages = fit;
  if (lay.stages < 1) return LS_E_SIZE;
  lay.x_off = (uint32_t)lay.stages * STAGE_BYTES;
  lay.recv_off = lay.x_off + (uint32_t)x_bytes;
  lay.head_off = lay.recv_off + (uint32_t)recv_bytes;
  lay.bars_off = lay.head_off + (uint32_t)head_bytes;
  // the whole SM is asked for although less is used: a block of this kernel, resident early,
  // must not take room from the blocks of the kernel before it (measured: slower otherwise)
  lay.smem = MAX_DYNAMIC_SMEM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((N + BM - 1) / BM, (T + BN - 1) / BN, plan.shares);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = lay.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = plan.shares;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ls_dependent_launch ? 2 : 1;
  LS_COUNT(EPI == 3 ? LS_K_GEMM_TC_FEW_QKV : NORM ? LS_K_GEMM_TC_FEW_NORM : LS_K_GEMM_TC_FEW);
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_few_kernel<BN, EPI, TC, NORM>, mw, mx, norm, heads, (TC*)C, T, N,
                                     K, ldc, plan.kb_per_share, plan.shares, lay, err);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

template <int BN, int EPI, typename TC>
int launch_walk(const CUtensorMap& mw, const CUtensorMap& mx, void* C, int T, int N, int K, int64_t ldc,
                const Plan& plan, int* err, cudaStream_t stream) {
  using S = Shape<BN, EPI>;
  constexpr int EW = S::REGION_COLS > 128 ? 8 : 4;       // wide tiles need two epilogue warpgroups
  if constexpr (S::REGION_COLS <= 256) {
    static bool configured = false;
    if (!configured) {
      if (cudaFuncSetAttribute(gemm_tc_walk_kernel<BN, EPI, TC, EW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)S::SMEM) != cudaSuccess)
        return LS_E_SMEM;
      configured = true;
    }
    const int tiles_n = (N + BM - 1) / BM, tiles_t = (T + BN - 1) / BN;
    const int tiles = tiles_n * tiles_t;
    const int sms = sm_count();
    LS_COUNT(LS_K_GEMM_TC_WALK);
    ls_launch(gemm_tc_walk_kernel<BN, EPI, TC, EW>, tiles < sms ? tiles : sms, EW == 8 ? 320 : 192, S::SMEM,
              stream, mw, mx, (TC*)C, T, N, K, ldc, plan.kb_per_share, plan.shares, tiles_n, tiles, err);
    return ls_launch_status();
  } else {
    return LS_E_SIZE;
  }
}

// How many pairs of blocks the device runs at one time (0: pairs cannot be launched).
template <int EPI, int FN, typename TC>
int resident_pairs() {
  using S = RowsShape<EPI, FN, 2>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sm_count());
  cfg.blockDim = dim3(320);
  cfg.dynamicSmemBytes = S::SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int pairs = 0;
  if (cudaOccupancyMaxActiveClusters(&pairs, gemm_tc_rows_kernel<EPI, FN, 2, TC>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return pairs;
}

template <int EPI, int FN, int CTAS, typename TC>
int launch_rows(const CUtensorMap& mw, const CUtensorMap& mx, void* C, int T, int N, int K, int64_t ldc,
                const Plan& plan, int* err, cudaStream_t stream) {
  using S = RowsShape<EPI, FN, CTAS>;
  // bfloat16 outputs that are not added to leave by TMA stores, where the map can be made
  CUtensorMap mc = mx;
  int store_by_tma = 0;
  if (EPI != 1 && sizeof(TC) == 2 && ((uintptr_t)C & 15) == 0 && (ldc % 8) == 0 && make_map(&mc, C, T, N, ldc, 32))
    store_by_tma = 1;
  static bool configured = false;
  static int resident = 0;                       // blocks, or pairs of them, that run at one time
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_rows_kernel<EPI, FN, CTAS, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)S::SMEM) != cudaSuccess)
      return LS_E_SMEM;
    resident = CTAS == 2 ? resident_pairs<EPI, FN, TC>() : sm_count();
    configured = true;
  }
  if (resident <= 0) return LS_E_SIZE;
  const int tiles_t = (T + BM * CTAS - 1) / (BM * CTAS), tiles_n = (N + FN - 1) / FN;
  const int tiles = tiles_t * tiles_n;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(CTAS * (tiles < resident ? tiles : resident));
  cfg.blockDim = dim3(320);
  cfg.dynamicSmemBytes = S::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ls_dependent_launch ? 2 : 1;
  LS_COUNT(CTAS == 2 ? LS_K_GEMM_TC_ROWS_PAIR : LS_K_GEMM_TC_ROWS);
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_rows_kernel<EPI, FN, CTAS, TC>, mw, mx, mc, store_by_tma, (TC*)C, T,
                                     N, K, ldc, plan.kb_per_share, plan.shares, tiles_t, tiles, err);
  if (e != cudaSuccess) return (int)e;
  return ls_launch_status();
}

int rows_pairs = 1;     // 1: tiles of 256 tokens on pairs of blocks; 0: tiles of 128 tokens on single blocks

template <int EPI, int FN, typename TC>
int launch_rows_as(const CUtensorMap& mw, const CUtensorMap& mx, void* C, int T, int N, int K, int64_t ldc,
                   const Plan& plan, int* err, cudaStream_t stream) {
  if (rows_pairs) return launch_rows<EPI, FN, 2, TC>(mw, mx, C, T, N, K, ldc, plan, err, stream);
  return launch_rows<EPI, FN, 1, TC>(mw, mx, C, T, N, K, ldc, plan, err, stream);
}

// more than 128 tokens: the kernel with the tokens on the M side
int run_rows(const void* X, const void* W, void* C, int c_dtype, int T, int N, int K, int64_t ldx, int64_t ldw,
             int64_t ldc, int epilogue, const Plan& plan, int* err, cudaStream_t stream) {
  typedef __nv_bfloat16 bf16;
  if ((ldx % 8) || ((uintptr_t)X & 15)) return LS_E_ALIGN;
  CUtensorMap mw, mx;
  const int ctas = rows_pairs ? 2 : 1;
  // tiles of 256 features unless they would leave SMs without one (the tile's width changes no sum)
  const int tiles_t = (T + BM * ctas - 1) / (BM * ctas);
  const bool wide = epilogue != 2 && tiles_t * ((N + 255) / 256) * ctas >= sm_count();
  // a block's box of weight rows: the tile's (silu-mul: its gate rows, then its up rows), half of them in a pair
  const int box = epilogue == 2 ? 128 : (wide ? 256 : 128) / ctas;
  if (!make_map(&mw, W, epilogue == 2 ? 2 * N : N, K, ldw, box)) return LS_E_SIZE;
  if (!make_map(&mx, X, T, K, ldx, BM)) return LS_E_SIZE;
  if (epilogue == 2) {
    if (c_dtype == LS_BF16) return launch_rows_as<2, 128, bf16>(mw, mx, C, T, N, K, ldc, plan, err, stream);
    return LS_E_DTYPE;
  }
  if (epilogue == 0 && c_dtype == LS_BF16)
    return wide ? launch_rows_as<0, 256, bf16>(mw, mx, C, T, N, K, ldc, plan, err, stream)
                : launch_rows_as<0, 128, bf16>(mw, mx, C, T, N, K, ldc, plan, err, stream);
  if (epilogue == 0 && c_dtype == LS_F32)
    return wide ? launch_rows_as<0, 256, float>(mw, mx, C, T, N, K, ldc, plan, err, stream)
                : launch_rows_as<0, 128, float>(mw, mx, C, T, N, K, ldc, plan, err, stream);
  if (epilogue == 1 && c_dtype == LS_F32)
    return wide ? launch_rows_as<1, 256, float>(mw, mx, C, T, N, K, ldc, plan, err, stream)
                : launch_rows_as<1, 128, float>(mw, mx, C, T, N, K, ldc, plan, err, stream);
  return LS_E_DTYPE;
}

// norm == nullptr: the token operand is read through `mx`; heads: the q/k/v epilogue's targets
template <int BN, int EPI, typename TC>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const NormArgs* norm, const LsQkvStore* heads, void* C, int T,
           int N, int K, int64_t ldc, const Plan& plan, int* err, cudaStream_t stream) {
  if constexpr (EPI == 3) {
    if constexpr (BN <= 32) {
      if (!plan.in_cluster || heads == nullptr) return LS_E_SIZE;
      NormArgs none = {};
      if (norm != nullptr) return launch_few<BN, 3, TC, true>(mw, mx, *norm, *heads, C, T, N, K, ldc, plan, err, stream);
      return launch_few<BN, 3, TC, false>(mw, mx, none, *heads, C, T, N, K, ldc, plan, err, stream);
    } else {
      return LS_E_SIZE;
    }
  } else {
    if (!plan.in_cluster) return launch_walk<BN, EPI, TC>(mw, mx, C, T, N, K, ldc, plan, err, stream);
    if constexpr (BN <= 32) {
      LsQkvStore no_heads = {};
      if (norm != nullptr)
        return launch_few<BN, EPI, TC, true>(mw, mx, *norm, no_heads, C, T, N, K, ldc, plan, err, stream);
      NormArgs none = {};
      return launch_few<BN, EPI, TC, false>(mw, mx, none, no_heads, C, T, N, K, ldc, plan, err, stream);
    } else if constexpr (BN <= 128) {
      if (norm != nullptr) return LS_E_SIZE;
      return launch_cluster<BN, EPI, TC>(mw, mx, C, T, N, K, ldc, plan, err, stream);
    } else {
      return LS_E_SIZE;
    }
  }
}

template <int BN>
int dispatch(const CUtensorMap& mw, const CUtensorMap& mx, const NormArgs* norm, const LsQkvStore* heads, void* C,
             int c_dtype, int T, int N, int K, int64_t ldc, int epilogue, const Plan& plan, int* err,
             cudaStream_t stream) {
  typedef __nv_bfloat16 bf16;
  if (epilogue == 0 && c_dtype == LS_BF16)
    return launch<BN, 0, bf16>(mw, mx, norm, heads, C, T, N, K, ldc, plan, err, stream);
  if (epilogue == 0 && c_dtype == LS_F32)
    return launch<BN, 0, float>(mw, mx, norm, heads, C, T, N, K, ldc, plan, err, stream);
  if (epilogue == 1 && c_dtype == LS_F32)
    return launch<BN, 1, float>(mw, mx, norm, heads, C, T, N, K, ldc, plan, err, stream);
  if (epilogue == 2 && c_dtype == LS_BF16) {
    if constexpr (BN <= 128) return launch<BN, 2, bf16>(mw, mx, norm, heads, C, T, N, K, ldc, plan, err, stream);
  }
  if (epilogue == 3 && c_dtype == LS_BF16)
    return launch<BN, 3, bf16>(mw, mx, norm, heads, C, T, N, K, ldc, plan, err, stream);
  return LS_E_DTYPE;
}

int run(const void* X, const NormArgs* norm, const LsQkvStore* heads, const void* W, void* C, int c_dtype, int T,
        int N, int K, int64_t ldx, int64_t ldw, int64_t ldc, int epilogue, int* err, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0 || epilogue < 0 || epilogue > 3 || (epilogue == 3) != (heads != nullptr)) return LS_E_SIZE;
  if ((K % 8) || (ldw % 8)) return LS_E_ALIGN;     // 16-byte row pitch
  if ((uintptr_t)W & 15) return LS_E_ALIGN;
  if ((N + BM - 1) / BM > 2147483647 / 2 || (T + 15) / 16 > 65535) return LS_E_SIZE;
  const Plan plan = make_plan(T, N, K, epilogue);
  const int bn = plan.bn;
  if (epilogue == 3 && (!plan.in_cluster || bn > 32)) return LS_E_SIZE;    // before any work is done
  if (T > 128) {
    if (norm != nullptr || epilogue == 3) return LS_E_SIZE;
    return run_rows(X, W, C, c_dtype, T, N, K, ldx, ldw, ldc, epilogue, plan, err, stream);
  }
  const int w_rows = epilogue == 2 ? 2 * N : N;
  CUtensorMap mw, mx;
  if (!make_map(&mw, W, w_rows, K, ldw, BM)) return LS_E_SIZE;
  if (norm == nullptr) {
    if ((ldx % 8) || ((uintptr_t)X & 15)) return LS_E_ALIGN;
    if (!make_map(&mx, X, T, K, ldx, bn)) return LS_E_SIZE;
  } else {
    // the fused form serves the cluster kernel only, up to 32 tokens (every block of the
    // cluster norms all rows again, which pays only while they are few), and only while
    // the normed rows of one share fit their shared-memory budget
    if (!plan.in_cluster || bn > 32 || plan.kb_per_share * bn * 128 > NORM_X_BYTES) return LS_E_SIZE;
    if ((K % 4) || ((uintptr_t)norm->h & 15) || ((uintptr_t)norm->gain & 15)) return LS_E_ALIGN;
    mx = mw;
  }
  switch (bn) {
    case 16: return dispatch<16>(mw, mx, norm, heads, C, c_dtype, T, N, K, ldc, epilogue, plan, err, stream);
    case 32: return dispatch<32>(mw, mx, norm, heads, C, c_dtype, T, N, K, ldc, epilogue, plan, err, stream);
    case 64: return dispatch<64>(mw, mx, norm, heads, C, c_dtype, T, N, K, ldc, epilogue, plan, err, stream);
    case 128: return dispatch<128>(mw, mx, norm, heads, C, c_dtype, T, N, K, ldc, epilogue, plan, err, stream);
  }
  return LS_E_SIZE;
}

}  // namespace

LS_API void ls_set_dependent_launch_tc(int on) { ls_dependent_launch = on ? 1 : 0; }

LS_API const char* ls_constants_gemm_tc() {
  static char buf[512];
  static const LsConstant c[] = {{"gemm_tc.weight_rows_per_tile", BM}, {"gemm_tc.k_block", BK},
                                 {"gemm_tc.share_rule.blocks_per_round", LS_SHARE_RULE_BLOCKS},
                                 {"gemm_tc.share_rule.fixed_cost", LS_SHARE_RULE_FIXED},
                                 {"gemm_tc.share_rule.min_depth", LS_SHARE_RULE_MIN_DEPTH},
                                 {"gemm_tc.share_rule.max_shares", LS_SHARE_RULE_MAX_SHARES},
                                 {"gemm_tc.few_tokens_norm_bytes", NORM_X_BYTES}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}

// launches of this library's kernels so far, in the order of LS_KERNEL_NAMES
LS_API const char* ls_kernel_names_tc() { return LS_KERNEL_NAMES; }
LS_API int ls_kernel_launches_tc(unsigned long long* out, int n) {
  for (int i = 0; i < n && i < LS_K_COUNT; ++i) out[i] = ls_kernel_launches[i];
  return LS_K_COUNT;
}

// Whether products of more than 128 tokens run on pairs of blocks (the default) or on single
// blocks; the sums are the same either way.
LS_API void ls_set_gemm_tc_pairs(int on) { rows_pairs = on ? 1 : 0; }

// The token tile for T tokens of a product with an (N, K) weight (it does not change any sum).
LS_API int ls_gemm_tc_token_tile(int T, int N, int K, int epilogue) {
  return make_plan(T, N, K, epilogue).bn;
}

// X [T, K] and W [N, K] (or [2N, K] for silu-mul) bfloat16 with row pitches ldx,
// ldw; C [T, N].  Refuses (LS_E_ALIGN, LS_E_SIZE) what TMA cannot address, so
// that the caller can use the CUDA-core product instead.
LS_API int ls_gemm_nt_tc(const void* X, const void* W, void* C, int c_dtype, int T, int N, int K,
                         int64_t ldx, int64_t ldw, int64_t ldc, int epilogue, int* err,
                         cudaStream_t stream) {
  if (epilogue == 3) return LS_E_SIZE;
  return run(X, nullptr, nullptr, W, C, c_dtype, T, N, K, ldx, ldw, ldc, epilogue, err, stream);
}

// The same product with the token operand made in the kernel:
// X[t, :] = rmsnorm(h[row_index ? row_index[t] : t, :]) with `gain` and `eps`, bit for bit
// what ls_rmsnorm writes.  h [src_rows, K] float32.  Serves few tokens (the cluster form);
// returns LS_E_SIZE or LS_E_ALIGN, having launched nothing, where it does not apply, and
// the caller then runs ls_rmsnorm and ls_gemm_nt_tc.
LS_API int ls_gemm_nt_tc_rmsnorm(const float* h, const int* row_index, int src_rows, const void* gain,
                                 int gain_dtype, float eps, const void* W, void* C, int c_dtype, int T,
                                 int N, int K, int64_t ldw, int64_t ldc, int epilogue, int* err,
                                 cudaStream_t stream) {
  if (gain_dtype != LS_F32 && gain_dtype != LS_BF16) return LS_E_DTYPE;
  NormArgs norm;
  norm.h = h;
  norm.row_index = row_index;
  norm.gain = gain;
  norm.gain_bf16 = gain_dtype == LS_BF16 ? 1 : 0;
  norm.src_rows = src_rows;
  norm.eps = eps;
  if (epilogue == 3) return LS_E_SIZE;
  return run(nullptr, &norm, nullptr, W, C, c_dtype, T, N, K, 0, ldw, ldc, epilogue, err, stream);
}

// The q/k/v projection of few tokens with its heads finished in the epilogue: what
// ls_gemm_nt_tc (or ls_gemm_nt_tc_rmsnorm when h is given instead of X) followed by
// ls_qk_norm_rope_store writes, bit for bit, without the projection going through memory.
// W [(nq + 2 nkv) * d, K]; the head size must divide 128.  Returns LS_E_SIZE or LS_E_ALIGN,
// having launched nothing, where it does not apply (more than 32 tokens, a weight whose depth
// is not shared out); the caller then runs the two kernels.
LS_API int ls_gemm_nt_tc_qkv_heads(const void* X, int64_t ldx, const float* h, const int* row_index, int src_rows,
                                   const void* gain, int gain_dtype, float eps, const void* W, int64_t ldw, int T,
                                   int K, void* q_out, void* pages, const void* q_gain, const void* k_gain,
                                   int head_gain_dtype, const float* cos_table, const float* sin_table,
                                   const int* positions, const int* token_req, const int* block_table,
                                   int table_stride, int nq, int nkv, int d, int rot_dim, int page_size,
                                   int num_pages, int max_positions, float head_eps, int write_cache, int* err,
                                   cudaStream_t stream) {
  if (d <= 0 || BM % d || nq <= 0 || nkv <= 0) return LS_E_SIZE;
  if (rot_dim < 0 || rot_dim > d || (rot_dim & 1)) return LS_E_SIZE;
  if (head_gain_dtype != LS_F32 && head_gain_dtype != LS_BF16) return LS_E_DTYPE;
  LsQkvStore heads;
  heads.q_out = q_out;
  heads.pages = pages;
  heads.q_gain = q_gain;
  heads.k_gain = k_gain;
  heads.cos_table = cos_table;
  heads.sin_table = sin_table;
  heads.positions = positions;
  heads.token_req = token_req;
  heads.block_table = block_table;
  heads.gain_bf16 = head_gain_dtype == LS_BF16 ? 1 : 0;
  heads.table_stride = table_stride;
  heads.nq = nq;
  heads.nkv = nkv;
  heads.d = d;
  heads.rot_dim = rot_dim;
  heads.page_size = page_size;
  heads.num_pages = num_pages;
  heads.max_positions = max_positions;
  heads.write_cache = write_cache;
  heads.eps = head_eps;
  heads.interleaved = 0;     // the caller takes rotations of neighbouring pairs to the kernel of their own
  const int N = (nq + 2 * nkv) * d;
  if (h == nullptr) return run(X, nullptr, &heads, W, nullptr, LS_BF16, T, N, K, ldx, ldw, 0, 3, err, stream);
  if (gain_dtype != LS_F32 && gain_dtype != LS_BF16) return LS_E_DTYPE;
  NormArgs norm;
  norm.h = h;
  norm.row_index = row_index;
  norm.gain = gain;
  norm.gain_bf16 = gain_dtype == LS_BF16 ? 1 : 0;
  norm.src_rows = src_rows;
  norm.eps = eps;
  return run(nullptr, &norm, &heads, W, nullptr, LS_BF16, T, N, K, 0, ldw, 0, 3, err, stream);
}
