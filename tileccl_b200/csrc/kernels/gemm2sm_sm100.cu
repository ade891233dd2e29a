// Plain GEMM on CTA pairs: C[M, N] = A[M, K] @ B, 16-bit inputs, fp32 accumulation in TMEM.
//
// Two CTAs (a cluster of two, on neighbouring SMs) work on one 256 x 256 tile of C with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and its own 128 of the
// 256 columns of B, the tensor cores of both SMs read both halves of B, and each CTA ends
// up with its 128 x 256 part of the accumulator in its own TMEM.  Against the one-CTA
// kernel (gemm_sm100.cu) a K block costs 32 KB instead of 48 KB of shared-memory fill per
// SM, so the operand ring is six stages deep instead of four and the L2 -> SM traffic per
// FLOP drops by a third; that fill, not the tensor pipe, is what bounds the one-CTA form.
//
// Roles per CTA (256 threads): warp 0 TMA producer (own halves; the byte counts of both
// CTAs land on the leader's "full" barrier), warp 1 MMA issuer (leader CTA only), warp 2
// TMEM allocation, warps 4-7 epilogue (own 128 rows).  No operand load uses multicast.
// Every wait is bounded; both CTAs always reach the closing cluster barrier.
#include "device/ptx.cuh"
#include "device/tile_compute.cuh"
#include "kernels/gemm_sm100.cuh"

namespace tileccl {

namespace {

constexpr int kPairStages = 6;
constexpr int kPairStageABytes = kBM * kBK * 2;          // 16 KiB: 128 rows x 64 K
constexpr int kPairStageBBytes = (kBN / 2) * kBK * 2;    // 16 KiB: 128 of the 256 columns
constexpr int kPairStageBytes = kPairStageABytes + kPairStageBBytes;
constexpr int kPairSmemPipe = kPairStages * kPairStageBytes;
static_assert(kPairSmemPipe == kSmemPipe, "both kernels use the same shared-memory budget");

__device__ __forceinline__ void tma_store_3d_pair(const CUtensorMap* m, int x, int y, int z,
                                                  uint32_t smem_src) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::
          "l"(reinterpret_cast<uint64_t>(m)),
      "r"(x), "r"(y), "r"(z), "r"(smem_src)
      : "memory");
}

}  // namespace

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm2sm_sm100_kernel(const __grid_constant__ FusedGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_epi = smem_base + kPairSmemPipe;
  const uint32_t smem_ctl = smem_epi + kSmemEpi;
  uint8_t* ctl_generic = smem_raw + (smem_ctl - smem_u32(smem_raw));

  const uint32_t bar_full = smem_ctl;                              // kPairStages x 8 B (leader's are used)
  const uint32_t bar_empty = bar_full + 8 * kPairStages;           // kPairStages x 8 B (one set per CTA)
  const uint32_t bar_acc_full = bar_empty + 8 * kPairStages;       // kAccBufs x 8 B (one set per CTA)
  const uint32_t bar_acc_empty = bar_acc_full + 8 * kAccBufs;      // kAccBufs x 8 B (leader's are used)
  const uint32_t bar_drain = bar_acc_empty + 8 * kAccBufs;         // 8 B
  const uint32_t tmem_slot = bar_drain + 8;                        // 4 B
  static_assert(8 * (2 * kPairStages + 2 * kAccBufs + 1) + 8 <= kSmemCtl, "control block overflow");
  volatile uint32_t* tmem_slot_g =
      reinterpret_cast<volatile uint32_t*>(ctl_generic + (tmem_slot - smem_ctl));
  volatile uint32_t* abort_flag = tmem_slot_g + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();        // 0 = leader
  const bool leader = cta == 0;
  uint32_t* status = reinterpret_cast<uint32_t*>(p.status);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);            // the leader's arrive.expect_tx
      mbar_init(bar_empty + 8 * s, 1);           // one multicast commit
    }
    for (int a = 0; a < kAccBufs; ++a) {
      mbar_init(bar_acc_full + 8 * a, 1);        // one multicast commit
      mbar_init(bar_acc_empty + 8 * a, 2 * kEpiWarps);   // epilogue warps of both CTAs
    }
    mbar_init(bar_drain, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, kAccBufs * kBN);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                            // barriers and TMEM of both CTAs exist
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_g;

  WaitBudget wb;
  wb.start(p.wait_budget_ns, abort_flag);

  // Pair-tiles (256 x 256) in row-major order; the pair takes every (gridDim.x / 2)-th one.
  const int pair = static_cast<int>(blockIdx.x >> 1);
  const int n_pairs = static_cast<int>(gridDim.x >> 1);
  const int m2_tiles = (p.m_tiles_local + 1) / 2;
  const int total = m2_tiles * p.n_tiles_local;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one_sync()) {
      tma_prefetch_desc(&p.tma_a);
      tma_prefetch_desc(&p.tma_b_half);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = pair; ok && t < total; t += n_pairs) {
        const int lm2 = t / p.n_tiles_local, ln = t - lm2 * p.n_tiles_local;
        const int a_row0 = (lm2 * 2 + static_cast<int>(cta)) * kBM;
        const int b_col0 = ln * kBN + static_cast<int>(cta) * (kBN / 2);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, wb)) {
            report_status(status, kStatusTimeoutMbarrier, 71, 0, 0, cta, t);
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * kPairStageBytes;
          const uint32_t sb = sa + kPairStageABytes;
          // Bytes of both CTAs are counted on the leader's barrier.
          if (leader) mbar_expect_tx(bar_full + 8 * stage, 2 * kPairStageBytes);
          const uint32_t bar = mapa_shared(bar_full + 8 * stage, 0);
          tma_load_2d_pair(sa, &p.tma_a, kb * kBK, a_row0, bar);
          if (p.b_kmajor) {
            tma_load_2d_pair(sb, &p.tma_b_half, kb * kBK, b_col0, bar);
          } else {
#pragma unroll
            for (int i = 0; i < kBN / 2 / 64; ++i)
              tma_load_2d_pair(sb + i * (64 * kBK * 2), &p.tma_b_half, b_col0 + i * 64, kb * kBK,
                               bar);
          }
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1 && leader) {
    // ------------------------- MMA issuer (leader CTA) -------------------------
    if (elect_one_sync()) {
      const uint32_t idesc = umma_idesc_f16(p.is_bf16, 0, p.b_kmajor ? 0 : 1, 2 * kBM, kBN);
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      for (int t = pair; ok && t < total; t += n_pairs) {
        if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, wb)) {
          report_status(status, kStatusTimeoutMbarrier, 72, 0, 0, cta, t);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, wb)) {
            report_status(status, kStatusTimeoutMbarrier, 73, 0, 0, cta, t);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * kPairStageBytes;
          const uint32_t sb = sa + kPairStageABytes;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t da = umma_smem_desc_sw128(sa + k * (kUmmaK * 2), 16, 1024);
            const uint64_t db =
                p.b_kmajor ? umma_smem_desc_sw128(sb + k * (kUmmaK * 2), 16, 1024)
                           : umma_smem_desc_sw128(sb + k * (kUmmaK * 128), 64 * kBK * 2, 1024);
            umma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(bar_empty + 8 * stage, 3);     // frees the stage in both CTAs
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(bar_acc_full + 8 * acc, 3);      // accumulators complete in both CTAs
        if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) {
        // Outstanding MMAs must finish before TMEM is released.
        umma_commit_pair(bar_drain, 1);
        for (int it = 0; it < 1000000 && !mbar_try_wait(bar_drain, 0); ++it) {}
      }
    }
  } else if (warp >= 4) {
    // -------------------------------- epilogue --------------------------------
    const int q = warp - 4;
    const bool bf16 = p.is_bf16 != 0;
    const uint32_t my_epi = smem_epi + q * (kEpiBufs * kEpiBufBytes);
    const uint32_t leader_acc_empty = mapa_shared(bar_acc_empty, 0);
    uint32_t acc = 0, acc_phase = 0;
    uint32_t buf = 0;
    for (int t = pair; t < total; t += n_pairs) {
      const int lm2 = t / p.n_tiles_local, ln = t - lm2 * p.n_tiles_local;
      const int out_y = (lm2 * 2 + static_cast<int>(cta)) * kBM;
      const int out_x = ln * kBN;
      if (!mbar_wait(bar_acc_full + 8 * acc, acc_phase, wb)) {
        if (lane == 0) report_status(status, kStatusTimeoutMbarrier, 74, 0, 0, cta, t);
        break;
      }
      tcgen05_fence_after();
      const uint32_t t_acc = tmem_base + acc * kBN + (static_cast<uint32_t>(q * 32) << 16);
      for (int ch = 0; ch < kBN / kChunkN; ++ch) {
        float v[kChunkN];
        {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(t_acc + ch * kChunkN, r0);
          tmem_ld_32x32b_x32(t_acc + ch * kChunkN + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v[i] = __uint_as_float(r0[i]);
            v[32 + i] = __uint_as_float(r1[i]);
          }
        }
        if (ch == kBN / kChunkN - 1) {
          // Every TMEM read of this accumulator is done: tell the leader's MMA warp.
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(leader_acc_empty + 8 * acc);
        }
        if (lane == 0) tma_store_wait_read<kEpiBufs - 1>();
        __syncwarp();
        const uint32_t sbuf = my_epi + buf * kEpiBufBytes;
#pragma unroll
        for (int j = 0; j < kChunkN / 8; ++j) {
          const uint4 w = tile_cast_f32x8(bf16, &v[j * 8]);
          const uint32_t addr = sbuf + lane * 128 + ((j ^ (lane & 7)) << 4);
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w.x), "r"(w.y),
                       "r"(w.z), "r"(w.w)
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d_pair(&p.tma_out[0], out_x + ch * kChunkN, out_y + q * kSlabM, 0, sbuf);
          tma_store_commit();
        }
        buf ^= 1u;
      }
      if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  // Neither CTA may retire while its partner can still read its operands or touch its
  // barriers; TMEM goes back only after every MMA and every TMEM read is done.
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, kAccBufs * kBN);
  }
}

cudaError_t launch_gemm2sm(const FusedGemmParams& p, int grid, cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !attr_set[dev]) {
    e = cudaFuncSetAttribute(gemm2sm_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemTotal);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  grid &= ~1;   // whole pairs only
  if (grid < 2) grid = 2;
  gemm2sm_sm100_kernel<<<grid, kThreads, kSmemTotal, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace tileccl
