// The state pass of the chunked Gated DeltaNet prefill on the 5th-generation tensor cores
// (tcgen05 + TMEM), sm_100a.  Included by gdn.cu inside its unnamed namespace (ScanParams, kC, kD).
//
// Same contract as gdn_chunk_state_kernel (one part of the joint state [S | A_hat^T | B_hat^T] per
// CTA, chunks of 64 tokens in order, operands parked by gdn_chunk_pre_kernel), but the products run
// TRANSPOSED so that the 128 feature rows are the M dimension and the state never leaves TMEM:
//     Xt     = X^T [dv x dk], fp32, 128 TMEM lanes x 128 columns (a summary's own layout)
//     D1     = Xt (-W)^T                [dv x 64]   A = a bf16 copy of Xt IN TMEM, B = -W tile (K-major)
//     Vnew^T = U^T + D1                 by the state threads (thread = TMEM lane = dv row), written back
//                                        to TMEM as bf16 pairs: Vnew^T and Vnew^T diag(e^(gc_last-gc))
//     D2a    = Xt Q^T,  D2b = Vnew^T P^T   [dv x 64]   (part 0)   O^T = D2a diag(e^gc) + D2b
//     Xt    <- e^gc_last Xt + (Vnew^T diag) K     A from TMEM, B = K tile (MN-major), accumulated in place
// Every A operand comes from TMEM: shared memory only carries the B tiles and U.  (With the bf16 copy
// of Xt in shared memory -- 32 KB written per chunk with four-way bank conflicts, 64 KB read by the two
// products that use it -- two CTAs per SM ran 2.2x slower each: shared-memory bandwidth, not latency,
// was the limit of a chunk.)
// Per chunk the state threads read Xt once (bf16 copy for the next products, scaled fp32 back), the
// MMA warp issues 24 (part 0) or 12 products from one elected lane, loader warps fetch the next
// chunk's tiles into the other buffer.  mma.sync cannot do better here: the previous kernel ran at
// the same speed with 4 or 16 warps, with or without prefetch (tensor pipe 34 % active).
//
// Every mbarrier wait is bounded; on expiry the CTA raises an abort flag, all roles leave their
// loops, TMEM is freed and the kernel returns (the status word of ScanParams is optional).
// (gdn.cu includes tc05.cuh at file scope before this file.)

struct TcStateSmem {
  static constexpr int kBuf = 0;                       // two buffers of the chunk's tiles
  static constexpr int kW = 0;                         // -W [64][128] swizzled (B, K-major)
  static constexpr int kK = kW + kC * kD * 2;          // K  [64][128] swizzled (B, MN-major)
  static constexpr int kQ = kK + kC * kD * 2;          // Q  [64][128] swizzled (B, K-major)    part 0
  static constexpr int kP = kQ + kC * kD * 2;          // P  [64][64]  swizzled (B, K-major)    part 0
  static constexpr int kU = kP + kC * kC * 2;          // U  [64][128] plain rows (read by the state threads)
  static constexpr int kVec = kU + kC * kD * 2;        // e^gc [64], e^(gc_last-gc) [64] fp32
  static constexpr int kBufBytes = ((kVec + 2 * kC * 4 + 1023) / 1024) * 1024;
  static constexpr int kOut = kBuf + 2 * kBufBytes;    // 4 warps x [64 tokens][32 dv] bf16 (+16 B per row): output staging
  static constexpr int kOutRow = 32 * 2 + 16;
  static constexpr int kBar = kOut + 4 * kC * kOutRow;
  static constexpr int kTotal = kBar + 256;
  static_assert(kTotal <= 227 * 1024, "shared memory of the tcgen05 chunk state kernel");
};

enum TcStateBar : int { kSbFull = 0, kSbEmpty = 2, kSbXsReady = 4, kSbD1Done = 5, kSbAReady = 6, kSbMmaDone = 7, kSbCount = 8 };
constexpr int kTcStateThreads = 256;   // warps 0-3 state (TMEM lanes), 4 MMA, 5-7 loaders
constexpr int kTcStatePolls = 1 << 18;
// TMEM columns (448 used of the 512 allocated): Xt fp32, its bf16 copy (A operand), D1, the two output
// accumulators, the two A operands made from Vnew^T.  (Alternating pairs of output accumulators,
// written out while the next chunk's first product runs, were measured and were not faster.)
constexpr int kColXt = 0, kColXtB = 128, kColD1 = 192, kColD2a = 256, kColD2b = 320, kColA1 = 384, kColA2 = 416;

__global__ void __launch_bounds__(kTcStateThreads, 1) gdn_chunk_state_tc_kernel(const __grid_constant__ ScanParams p) {
  using Sm = TcStateSmem;
  extern __shared__ __align__(1024) unsigned char tsm[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t sb = smem_u32(tsm);
  const uint32_t bar_base = sb + Sm::kBar;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tsm + Sm::kBar + kSbCount * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tsm + Sm::kBar + kSbCount * 8 + 8);
  auto bar = [&](int slot) { return bar_base + slot * 8; };
  const int part = blockIdx.x;
  const int h = blockIdx.y;
  const int r = blockIdx.z;
  const int t_begin = p.seg_off[r];
  const int t_end = p.seg_off[r + 1];
  const int n_chunks = (t_end - t_begin + kC - 1) / kC;
  const int64_t head_off = static_cast<int64_t>(h) * kD * kD;
  const int64_t hN = static_cast<int64_t>(h) * p.num_tokens;

  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(kSbFull + b), 3);     // one arrival per loader warp
      mbar_init(bar(kSbEmpty + b), 5);    // four state warps + the commit of the last product that read it
    }
    mbar_init(bar(kSbXsReady), 4);
    mbar_init(bar(kSbD1Done), 1);
    mbar_init(bar(kSbAReady), 4);
    mbar_init(bar(kSbMmaDone), 1);
    mbar_fence_init();
    *abort_flag = 0;
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  bool dead = false;
  auto wait = [&](int slot, uint32_t parity) -> bool {
    if (dead) return false;
    const uint32_t b = bar(slot);
    for (int i = 0; i < kTcStatePolls; ++i) {
      if (mbar_try_wait(b, parity & 1u)) return true;   // (a suspend-time hint, or spinning on test_wait, were both slower)
      if ((i & 63) == 63 && *abort_flag != 0) break;
    }
    dead = true;
    if (*abort_flag == 0 && p.status != nullptr) report(p.status, VA_DEV_WAIT_EXPIRED);
    *abort_flag = 1;
    return false;
  };
  auto wait_warp = [&](int slot, uint32_t parity) -> bool {
    const bool ok = __all_sync(0xffffffffu, wait(slot, parity));
    if (!ok) dead = true;
    return ok;
  };

  if (warp >= 5) {
    // ================================================================= loaders
    const int lt = tid - 5 * 32;
    for (int c = 0; c < n_chunks && !dead; ++c) {
      const int b = c & 1;
      const int t0 = t_begin + c * kC;
      if (!wait(kSbEmpty + b, ((c >> 1) & 1u) ^ 1u)) break;
      const uint32_t base = sb + Sm::kBuf + b * Sm::kBufBytes;
      // a [64][row_elems] bf16 tile of the scratch into a 128-byte-swizzled tile
      auto copy_sw = [&](uint32_t dst, const __nv_bfloat16* src, int row_elems) {
        const int per_row = row_elems >> 3;
        for (int idx = lt; idx < kC * per_row; idx += 96) {
          const int i = idx / per_row, ch = idx - i * per_row;
          const bool live = t0 + i < t_end;
          cp_async16(dst + sw_off(i, ch, kC), src + (hN + (live ? t0 + i : t0)) * row_elems + ch * 8, live ? 16 : 0);
        }
      };
      copy_sw(base + Sm::kW, p.s_w, kD);
      copy_sw(base + Sm::kK, p.s_k, kD);
      if (part == 0) {
        copy_sw(base + Sm::kQ, p.s_q, kD);
        copy_sw(base + Sm::kP, p.s_p, kC);
      }
      if (part != 1) {
        for (int idx = lt; idx < kC * (kD >> 3); idx += 96) {
          const int i = idx >> 4, ch = idx & 15;
          const bool live = t0 + i < t_end;
          cp_async16(base + Sm::kU + (i * kD + ch * 8) * 2, p.s_u + (hN + (live ? t0 + i : t0)) * kD + ch * 8, live ? 16 : 0);
        }
      }
      float* vec = reinterpret_cast<float*>(tsm + Sm::kBuf + b * Sm::kBufBytes + Sm::kVec);
      for (int i = lt; i < 2 * kC; i += 96) {
        const int j = i & (kC - 1);
        const bool live = t0 + j < t_end;
        const float* src = i < kC ? p.s_eg : p.s_ed;
        vec[i] = live ? src[hN + t0 + j] : 0.f;
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kSbFull + b));
    }
    cp_async_wait<0>();
  } else if (warp == 4) {
    // ================================================================= MMA issuer (converged warp)
    const uint32_t elected = elect_one();
    const uint32_t idesc_n64 = instr_desc(kC, false);
    const uint32_t idesc_n128 = instr_desc(kD, true);
    for (int c = 0; c < n_chunks; ++c) {
      const int b = c & 1;
      const uint32_t base = sb + Sm::kBuf + b * Sm::kBufBytes;
      if (!wait_warp(kSbFull + b, (c >> 1) & 1u)) break;
      if (!wait_warp(kSbXsReady, c & 1u)) break;
      tc_fence_after();
      const uint64_t w_desc = smem_desc(base + Sm::kW, 16, 1024);
      const uint64_t q_desc = smem_desc(base + Sm::kQ, 16, 1024);
      const uint64_t p_desc = smem_desc(base + Sm::kP, 16, 1024);
      const uint64_t k_desc = smem_desc(base + Sm::kK, kC * 128, 1024);   // MN-major view
      // D1 = Xt (-W)^T : panel ks / 4, 32 bytes per step inside it
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks)
        umma_ts(elected, tmem_base + kColD1, tmem_base + kColXtB + ks * 8,
                w_desc + static_cast<uint64_t>((ks >> 2) * (kC * 8) + (ks & 3) * 2), idesc_n64, ks > 0);
      umma_commit(elected, bar(kSbD1Done));
      if (part == 0) {
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks)
          umma_ts(elected, tmem_base + kColD2a, tmem_base + kColXtB + ks * 8,
                  q_desc + static_cast<uint64_t>((ks >> 2) * (kC * 8) + (ks & 3) * 2), idesc_n64, ks > 0);
      }
      if (!wait_warp(kSbAReady, c & 1u)) break;
      tc_fence_after();
      if (part == 0) {
#pragma unroll
        for (int ks = 0; ks < kC / 16; ++ks)
          umma_ts(elected, tmem_base + kColD2b, tmem_base + kColA1 + ks * 8, p_desc + static_cast<uint64_t>(ks * 2),
                  idesc_n64, ks > 0);
      }
#pragma unroll
      for (int ks = 0; ks < kC / 16; ++ks)
        umma_ts(elected, tmem_base + kColXt, tmem_base + kColA2 + ks * 8, k_desc + static_cast<uint64_t>(ks * 128),
                idesc_n128, true);
      umma_commit(elected, bar(kSbMmaDone));
      umma_commit(elected, bar(kSbEmpty + b));
    }
    dead = __any_sync(0xffffffffu, dead);
  } else {
    // ================================================================= state threads (thread = dv row)
    const int L = tid;                                                      // TMEM lane = row of Xt
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const bool sum_bf16 = part != 0 && p.summary_bf16 != 0;
    // ---- initial state into TMEM
    {
      const void* src = nullptr;
      if (part == 0) src = p.state0;
      else src = reinterpret_cast<const void*>(part == 1 ? p.init_a[r] : p.init_b[r]);
#pragma unroll
      for (int q0 = 0; q0 < kD; q0 += 32) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = (part == 1 && q0 + i == L) ? 1.f : 0.f;
        if (src != nullptr) {
          if (part == 0) {   // state0 [dk][dv]: column L
            const float* s0 = p.state0 + (static_cast<int64_t>(r) * p.num_v_heads + h) * kD * kD;
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = s0[(q0 + i) * kD + L];
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 x = sum_ld4(src, head_off + static_cast<int64_t>(L) * kD + q0 + i, sum_bf16);
              v[i] = x.x; v[i + 1] = x.y; v[i + 2] = x.z; v[i + 3] = x.w;
            }
          }
        }
        tmem_st32(lane_addr + kColXt + q0, v);
      }
      tc_fence_before();
    }
    // O^T of a chunk (part 0): read out of TMEM as soon as its products are done (bf16 pairs of
    // tokens 2i, 2i+1 of this thread's dv row), written to global memory later, off the chunk's
    // critical chain, through a per-warp staging tile so that the global stores are 16 bytes wide
    uint32_t o_pk[kC / 2];
    auto read_out = [&](const float* eg) {
#pragma unroll
      for (int q0 = 0; q0 < kC; q0 += 32) {
        float a[32], bq[32];
        tmem_ld32(lane_addr + kColD2a + q0, a);
        tmem_ld32(lane_addr + kColD2b + q0, bq);
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          o_pk[(q0 + i) >> 1] = pack_bf16(fmaf(a[i], eg[q0 + i], bq[i]), fmaf(a[i + 1], eg[q0 + i + 1], bq[i + 1]));
      }
    };
    auto store_out = [&](int t0) {
      unsigned char* stage = tsm + Sm::kOut + warp * (kC * Sm::kOutRow);
#pragma unroll
      for (int i = 0; i < kC / 2; ++i) {
        *reinterpret_cast<__nv_bfloat16*>(stage + (2 * i) * Sm::kOutRow + lane * 2) =
            __ushort_as_bfloat16(static_cast<unsigned short>(o_pk[i] & 0xffffu));
        *reinterpret_cast<__nv_bfloat16*>(stage + (2 * i + 1) * Sm::kOutRow + lane * 2) =
            __ushort_as_bfloat16(static_cast<unsigned short>(o_pk[i] >> 16));
      }
      __syncwarp();
      // 64 tokens x 64 bytes of this warp's 32 dv columns: 4 lanes per token, 8 tokens per pass
#pragma unroll
      for (int pass = 0; pass < kC / 8; ++pass) {
        const int j = pass * 8 + (lane >> 2);
        const int piece = lane & 3;
        const int tok = t0 + j;
        if (tok < t_end) {
          const uint4 v = *reinterpret_cast<const uint4*>(stage + j * Sm::kOutRow + piece * 16);
          *reinterpret_cast<uint4*>(p.out + (static_cast<int64_t>(tok) * p.num_v_heads + h) * kD + warp * 32 + piece * 8) = v;
        }
      }
      __syncwarp();
    };
    for (int c = 0; c < n_chunks && !dead; ++c) {
      const int b = c & 1;
      const int t0 = t_begin + c * kC;
      unsigned char* bufp = tsm + Sm::kBuf + b * Sm::kBufBytes;
      const float* eg = reinterpret_cast<const float*>(bufp + Sm::kVec);
      const float* ed = eg + kC;
      if (!wait_warp(kSbFull + b, (c >> 1) & 1u)) break;
      if (c > 0) {
        if (!wait_warp(kSbMmaDone, (c - 1) & 1u)) break;
        tc_fence_after();
        if (part == 0) read_out(reinterpret_cast<const float*>(tsm + Sm::kBuf + (b ^ 1) * Sm::kBufBytes + Sm::kVec));
        // the previous chunk's buffer is no longer read by these threads
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kSbEmpty + (b ^ 1)));
      }
      // ---- Xt: bf16 copy into TMEM (A operand of the next products), fp32 scaled by the chunk's
      //      total decay back in place (the state update accumulates on top of it)
      const int n_live = min(kC, t_end - t0);
      const float tail = eg[n_live - 1];   // tokens past the end do not decay the state
#pragma unroll
      for (int q0 = 0; q0 < kD; q0 += 32) {
        float v[32];
        tmem_ld32(lane_addr + kColXt + q0, v);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) pk[i >> 1] = pack_bf16(v[i], v[i + 1]);
        tmem_st16_issue(lane_addr + kColXtB + (q0 >> 1), pk);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= tail;
        tmem_st32(lane_addr + kColXt + q0, v);
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kSbXsReady));
      if (c > 0 && part == 0) store_out(t0 - kC);   // while the tensor core works on D1
      // ---- Vnew^T = U^T + D1 ; bf16 pairs of it and of its decayed form into TMEM (A operands)
      if (!wait_warp(kSbD1Done, c & 1u)) break;
      tc_fence_after();
      const __nv_bfloat16* Us = reinterpret_cast<const __nv_bfloat16*>(bufp + Sm::kU);
#pragma unroll
      for (int q0 = 0; q0 < kC; q0 += 32) {
        float v[32];
        tmem_ld32(lane_addr + kColD1 + q0, v);
        if (part != 1) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += __bfloat162float(Us[(q0 + i) * kD + L]);
        }
        uint32_t a1[16], a2[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          a1[i >> 1] = pack_bf16(v[i], v[i + 1]);
          a2[i >> 1] = pack_bf16(v[i] * ed[q0 + i], v[i + 1] * ed[q0 + i + 1]);
        }
        if (part == 0) tmem_st16_issue(lane_addr + kColA1 + (q0 >> 1), a1);
        tmem_st16_issue(lane_addr + kColA2 + (q0 >> 1), a2);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kSbAReady));
    }
    // ---- the last chunk's output rows, then the state
    if (!dead && n_chunks > 0) {
      const int c = n_chunks - 1;
      if (wait_warp(kSbMmaDone, c & 1u)) {
        tc_fence_after();
        if (part == 0)
        {
          read_out(reinterpret_cast<const float*>(tsm + Sm::kBuf + (c & 1) * Sm::kBufBytes + Sm::kVec));
          store_out(t_begin + c * kC);
        }
      }
    }
    if (!dead) {
      void* dst = nullptr;
      if (part == 0) dst = p.final_state;
      else dst = reinterpret_cast<void*>(part == 1 ? p.write_a[r] : p.write_b[r]);
      if (dst != nullptr) {
#pragma unroll
        for (int q0 = 0; q0 < kD; q0 += 32) {
          float v[32];
          tmem_ld32(lane_addr + kColXt + q0, v);
          if (part == 0) {
            float* fs = p.final_state + (static_cast<int64_t>(r) * p.num_v_heads + h) * kD * kD;
#pragma unroll
            for (int i = 0; i < 32; ++i) fs[(q0 + i) * kD + L] = v[i];
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              sum_st4(dst, head_off + static_cast<int64_t>(L) * kD + q0 + i, make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]), sum_bf16);
          }
        }
      }
      tc_fence_before();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
  }
}
