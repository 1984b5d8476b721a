// Dense contraction kernel for sm_100a:  D[b, m, n] = epilogue( sum_k A[b, m, k] * B[b, n, k] )
//
// One persistent CTA per SM, warp specialised:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of A and B tiles (128-byte swizzle)
//               into a B200_STAGES-deep shared-memory ring, completion on mbarriers
//   warp 1      owns tensor memory (tcgen05.alloc) and issues tcgen05.mma (kind::f16 or
//               kind::tf32, fp32 accumulators in TMEM); tcgen05.commit releases ring slots
//               and publishes finished accumulators
//   warps 2..   epilogue: tcgen05.ld of the accumulator (one TMEM lane = one output row per
//               thread), the routine's generated epilogue expression, global stores
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of
// tile i+1.  Every wait is bounded: a wait that does not complete within ~2 s raises the
// device status word, all roles drain and the CTA frees its tensor memory and returns.
//
// The translation unit that includes this text defines:
//   B200_GEMM_NAME            kernel symbol
//   B200_BM (128), B200_BN    tile extents (B200_BN multiple of 16, <= 256)
//   B200_BK                   k elements per ring slot (128 bytes worth)
//   B200_UMMA_K               k elements per tcgen05.mma (16 for 16-bit inputs, 8 for tf32)
//   B200_ELEM_BYTES           operand element size
//   B200_STAGES               ring depth
//   B200_EPI_WARPS            4, 8 or 16 (a multiple of 4: one warp per TMEM lane quarter and column part)
//   B200_STAGING_BYTES        bytes of one staging tile (32 rows x chunk columns of the widest output)
//   B200_STAGING_TILES        staging tiles per epilogue warp (2 when outputs leave as TMA stores and shared memory allows)
//   B200_EPI_PROLOGUE         declarations at the top of the epilogue role (pointers to the output tensor maps)
//   B200_LOAD_TILE_BYTES      bytes of the per-warp tile that receives a row operand's chunk by TMA (0: none)
//   B200_A_KMAJOR/B_KMAJOR    1: k is the contiguous axis of the operand, 0: m/n is
//   B200_IDESC                tcgen05 instruction descriptor (formats, majors, M, N)
//   B200_TMEM_COLS            power of two >= 2*B200_BN (and >= 32)
//   B200_EPI_PARAMS           extra kernel parameters (node pointers) of the epilogue
//   B200_EPILOGUE_ROW(...)    statement block evaluated per (row, 32-column chunk), see below
#ifndef B200_GEMM_SM100_CUH
#define B200_GEMM_SM100_CUH

#ifndef B200_TC_SM100_CUH
#include "tc_sm100.cuh"
#endif
struct b200_gemm_shape {
  unsigned int M, N, K;
  unsigned int B0, B1;          // batch extents, outer and inner (1 when absent)
  unsigned int a_b0, a_b1;      // 1 when the operand varies along that batch axis
  unsigned int b_b0, b_b1;
  unsigned int tiles_m, tiles_n;
  unsigned int tma_out;         // != 0: the epilogue's row-contiguous outputs leave as TMA stores (their maps are valid)
};


__device__ __forceinline__ void b200_tmem_ld_chunk(unsigned int taddr, unsigned int* r) {
#if B200_EPI_CHUNK == 64
  b200_tmem_ld32(taddr, r);
  b200_tmem_ld32(taddr + 32u, r + 32);
#elif B200_EPI_CHUNK == 32
  b200_tmem_ld32(taddr, r);
#else
  b200_tmem_ld16(taddr, r);
#endif
}

// Developer aid: with -DB200_TRACE, CTA 0 records nanoseconds since its start at a few points
// into words 2..15 of the device status buffer (printed by the host when B200_TRACE is set).
#ifdef B200_TRACE
#define B200_TR(slot) do { if (blockIdx.x == 0) status[slot] = (unsigned int)(b200_now_ns() - b200_t0); } while (0)
#else
#define B200_TR(slot) do { } while (0)
#endif

// per CTA: 128 rows of A; all of the tile's B columns, or half of them in pair mode
#define B200_CTA_M 128
#define B200_CTA_N (B200_BN / (1 + B200_CTA_PAIR))
#define B200_A_TILE_BYTES (B200_CTA_M * B200_BK * B200_ELEM_BYTES)
#define B200_B_TILE_BYTES (B200_CTA_N * B200_BK * B200_ELEM_BYTES)
#define B200_STAGE_BYTES (B200_A_TILE_BYTES + B200_B_TILE_BYTES)
#define B200_THREADS (64 + 32 * B200_EPI_WARPS)
// elements of the contiguous axis covered by one 128-byte swizzle row
#define B200_ROW_ELEMS (128 / B200_ELEM_BYTES)
#ifndef B200_EPI_CHUNK
#if B200_BN >= 32
#define B200_EPI_CHUNK 32
#else
#define B200_EPI_CHUNK 16
#endif
#endif
#ifndef B200_RASTER
#define B200_RASTER 8
#endif
// B200_SPLITK work units per tile, each over its own slice of the k blocks (the epilogue then adds
// its partial tile to the output with reductions in global memory)
#ifndef B200_SPLITK
#define B200_SPLITK 1
#endif

extern "C" __global__ void __launch_bounds__(B200_THREADS, 1)
B200_GEMM_NAME(const __grid_constant__ b200_tmap map_a, const __grid_constant__ b200_tmap map_b,
               const b200_gemm_shape shape, unsigned int* status B200_EPI_PARAMS) {
  extern __shared__ unsigned char b200_dyn_smem[];
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern
  const unsigned int smem_base = (b200_smem_addr(b200_dyn_smem) + 1023u) & ~1023u;
  unsigned char* smem_gen = b200_dyn_smem + (smem_base - b200_smem_addr(b200_dyn_smem));
  const unsigned int tiles_at = smem_base;
  // the epilogue warps' staging tiles follow the ring (1024-byte aligned, as the swizzled TMA stores want);
  // barriers and bookkeeping live after them
  unsigned long long* bars = (unsigned long long*)(smem_gen + B200_STAGES * B200_STAGE_BYTES +
                                                   B200_EPI_WARPS * (B200_STAGING_TILES * B200_STAGING_BYTES + B200_LOAD_TILE_BYTES));
  const unsigned int bar_full = b200_smem_addr(bars);                          // [STAGES]
  const unsigned int bar_empty = bar_full + 8u * B200_STAGES;                  // [STAGES]
  const unsigned int bar_acc_full = bar_empty + 8u * B200_STAGES;              // [2]
  const unsigned int bar_acc_empty = bar_acc_full + 16u;                       // [2]
  const unsigned int bar_load = bar_acc_empty + 16u;                           // [EPI_WARPS]: row operands loaded by TMA
  volatile unsigned int* tmem_slot = (volatile unsigned int*)(bars + 2 * B200_STAGES + 4 + B200_EPI_WARPS);
  volatile unsigned int* abort_flag = tmem_slot + 1;

  // the next kernel in the stream may be placed as soon as every CTA of this one is running
  asm volatile("griddepcontrol.launch_dependents;");
  const unsigned int warp = threadIdx.x >> 5;
  const unsigned int lane = threadIdx.x & 31u;
#ifdef B200_TRACE
  const unsigned long long b200_t0 = b200_now_ns();
  B200_TRE(-1);
#endif

  if (threadIdx.x == 32) {
    // the descriptors are fetched while the barriers and the tensor memory are being set up
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_b) : "memory");
  }
  if (threadIdx.x == 0) {
    for (unsigned int s = 0; s < B200_STAGES; ++s) {
      b200_mbar_init(bar_full + 8u * s, 1);
      b200_mbar_init(bar_empty + 8u * s, 1);
    }
    for (unsigned int a = 0; a < 2; ++a) {
      b200_mbar_init(bar_acc_full + 8u * a, 1);
      // the leader's accumulator buffer is free again when the epilogue warps of both CTAs are done with it
      b200_mbar_init(bar_acc_empty + 8u * a, B200_EPI_WARPS * (1 + B200_CTA_PAIR));
    }
    for (unsigned int w = 0; w < B200_EPI_WARPS; ++w) b200_mbar_init(bar_load + 8u * w, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc." B200_CG ".sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(b200_smem_addr((const void*)tmem_slot)),
                 "r"((unsigned int)B200_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit." B200_CG ".sync.aligned;" ::: "memory");
  }
  // set-up above touched no global memory; from here on the grids before this one must be complete
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  b200_cluster_sync();   // the peer's barriers are initialised before anything is signalled on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned int tmem_base = *tmem_slot;
  const unsigned int cta_rank = b200_cta_rank();
  // tiles are taken by CTA pairs in pair mode, by single CTAs otherwise
  const unsigned int worker = blockIdx.x / (1 + B200_CTA_PAIR), n_workers = gridDim.x / (1 + B200_CTA_PAIR);
  if (threadIdx.x == 0) B200_TR(2);   // set-up done

  const unsigned int tiles_per_batch = shape.tiles_m * shape.tiles_n;
  const unsigned int total_tiles = tiles_per_batch * shape.B0 * shape.B1;
  const unsigned int k_blocks = (shape.K + B200_BK - 1) / B200_BK;
  const unsigned int total_units = total_tiles * B200_SPLITK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      unsigned int slot = 0, phase = 0;
      bool live = true;
      for (unsigned int unit = worker; live && unit < total_units; unit += n_workers) {
        const unsigned int tile = unit % total_tiles, split = unit / total_tiles;
        const unsigned int kb0 = split * k_blocks / B200_SPLITK, kb1 = (split + 1u) * k_blocks / B200_SPLITK;
        const unsigned int bidx = tile / tiles_per_batch;
        const unsigned int t = tile - bidx * tiles_per_batch;
        // consecutive tiles walk down m first so that a wave of CTAs shares few B tiles
        const unsigned int group = t / (B200_RASTER * shape.tiles_n);
        const unsigned int first_m = group * B200_RASTER;
        const unsigned int rows = min((unsigned int)B200_RASTER, shape.tiles_m - first_m);
        const unsigned int r = t - group * B200_RASTER * shape.tiles_n;
        const unsigned int mt = first_m + r % rows;
        const unsigned int nt = r / rows;
        const unsigned int b0 = bidx / shape.B1, b1 = bidx - b0 * shape.B1;
        // this CTA's rows of A and its share of the tile's B columns
        const int m0 = (int)(mt * B200_BM + cta_rank * B200_CTA_M), n0 = (int)(nt * B200_BN + cta_rank * B200_CTA_N);
        for (unsigned int kb = kb0; kb < kb1; ++kb) {
#ifdef B200_INJECT_NO_LOADS
          // failure-detection test only: the producer loads nothing, so the waits for operands can
          // never be satisfied and must run out (no copy or MMA is ever in flight in this build)
          continue;
#endif
          if (!b200_wait(bar_empty + 8u * slot, phase ^ 1u, abort_flag, status, 1u)) { live = false; break; }
          // both CTAs' copies complete on the leader's barrier; the leader announces the bytes of both
          const unsigned int full = b200_map_to_cta(bar_full + 8u * slot, 0u);   // (the barrier itself when not paired)
          if (cta_rank == 0u) b200_mbar_expect_tx(bar_full + 8u * slot, B200_STAGE_BYTES * (1 + B200_CTA_PAIR));
          const unsigned int sa = tiles_at + slot * B200_STAGE_BYTES;
          const unsigned int sb = sa + B200_A_TILE_BYTES;
          const int k0 = (int)(kb * B200_BK);
#if B200_A_KMAJOR
          b200_tma_load_4d(sa, &map_a, full, k0, m0, (int)(b1 * shape.a_b1), (int)(b0 * shape.a_b0));
#else
#pragma unroll
          for (int c = 0; c < B200_CTA_M / B200_ROW_ELEMS; ++c)
            b200_tma_load_4d(sa + c * (B200_ROW_ELEMS * B200_BK * B200_ELEM_BYTES), &map_a, full, m0 + c * B200_ROW_ELEMS, k0,
                             (int)(b1 * shape.a_b1), (int)(b0 * shape.a_b0));
#endif
#if B200_B_KMAJOR
          b200_tma_load_4d(sb, &map_b, full, k0, n0, (int)(b1 * shape.b_b1), (int)(b0 * shape.b_b0));
#else
#pragma unroll
          for (int c = 0; c < B200_CTA_N / B200_ROW_ELEMS; ++c)
            b200_tma_load_4d(sb + c * (B200_ROW_ELEMS * B200_BK * B200_ELEM_BYTES), &map_b, full, n0 + c * B200_ROW_ELEMS, k0,
                             (int)(b1 * shape.b_b1), (int)(b0 * shape.b_b0));
#endif
          if (unit == worker && kb == kb0) B200_TR(3);   // first loads issued
          if (++slot == B200_STAGES) { slot = 0; phase ^= 1u; }
        }
      }
      B200_TR(4);   // producer done
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (the leader CTA of a pair)
    if (lane == 0 && cta_rank == 0u) {
      unsigned int slot = 0, phase = 0, acc = 0, acc_phase = 0;
      bool live = true;
      // operand descriptors of ring slot 0.  k-major: rows of 128 bytes, 8-row groups 1024 bytes
      // apart.  m/n-major: 64-element (128-byte) chunks of m/n, k rows 128 bytes apart, 8-row groups
      // 1024 bytes apart, chunks one box apart.
#if B200_A_KMAJOR
      const unsigned long long desc_a0 = b200_smem_desc(tiles_at, 16u, 1024u);
#else
      const unsigned long long desc_a0 = b200_smem_desc(tiles_at, B200_ROW_ELEMS * B200_BK * B200_ELEM_BYTES, B200_MN_GROUP_BYTES, B200_MN_SWIZZLE);
#endif
#if B200_B_KMAJOR
      const unsigned long long desc_b0 = b200_smem_desc(tiles_at + B200_A_TILE_BYTES, 16u, 1024u);
#else
      const unsigned long long desc_b0 =
          b200_smem_desc(tiles_at + B200_A_TILE_BYTES, B200_ROW_ELEMS * B200_BK * B200_ELEM_BYTES, B200_MN_GROUP_BYTES, B200_MN_SWIZZLE);
#endif
      for (unsigned int unit = worker; live && unit < total_units; unit += n_workers) {
        const unsigned int split = unit / total_tiles;
        const unsigned int kb0 = split * k_blocks / B200_SPLITK, kb1 = (split + 1u) * k_blocks / B200_SPLITK;
        if (!b200_wait(bar_acc_empty + 8u * acc, acc_phase ^ 1u, abort_flag, status, 2u)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned int d_tmem = tmem_base + acc * B200_BN;
        for (unsigned int kb = kb0; kb < kb1; ++kb) {
          if (!b200_wait(bar_full + 8u * slot, phase, abort_flag, status, 3u)) { live = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (unit == worker && kb == kb0) B200_TR(5);   // first operands landed
          // descriptors of this slot: the start-address field (bits 0-13, address >> 4) moves, the rest is fixed
          const unsigned long long da0 = desc_a0 + (unsigned long long)((slot * B200_STAGE_BYTES) >> 4);
          const unsigned long long db0 = desc_b0 + (unsigned long long)((slot * B200_STAGE_BYTES) >> 4);
#pragma unroll
          for (unsigned int ks = 0; ks < B200_BK / B200_UMMA_K; ++ks) {
            // a k step moves UMMA_K elements along a k-major row, or UMMA_K rows of 128 bytes in the m/n-major form
            const unsigned long long da = da0 + (unsigned long long)((ks * (B200_A_KMAJOR ? B200_UMMA_K * B200_ELEM_BYTES : B200_UMMA_K * 128u)) >> 4);
            const unsigned long long db = db0 + (unsigned long long)((ks * (B200_B_KMAJOR ? B200_UMMA_K * B200_ELEM_BYTES : B200_UMMA_K * 128u)) >> 4);
            b200_umma(d_tmem, da, db, (unsigned int)B200_IDESC, (kb != kb0 || ks != 0u) ? 1u : 0u);
          }
          b200_umma_commit(bar_empty + 8u * slot);  // frees the slot once these MMAs retire
          if (++slot == B200_STAGES) { slot = 0; phase ^= 1u; }
        }
        if (live) b200_umma_commit(bar_acc_full + 8u * acc);
        if (unit == worker) B200_TR(6);                  // tile 0 MMAs issued
        else if (unit == worker + n_workers) B200_TR(7); // tile 1 MMAs issued
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const unsigned int ew = warp - 2;                 // 0 .. EPI_WARPS-1
    const unsigned int quarter = warp & 3u;           // TMEM lanes this warp may read
    const unsigned int col_half = ew >> 2;            // which part of the tile's columns this warp owns
    const unsigned int cols_per_warp = B200_BN / (B200_EPI_WARPS / 4);
    // this warp's 4 KB staging tile (transposes a chunk so that stores cover whole row segments)
    uint4* b200_stage = (uint4*)(smem_gen + B200_STAGES * B200_STAGE_BYTES + ew * (unsigned int)(B200_STAGING_TILES * B200_STAGING_BYTES));
    b200_epi_state b200_es;
    b200_es.tma = shape.tma_out != 0u;
    b200_es.nst = 0u;
    // the tile and barrier of a row operand that arrives by TMA (B200_LOAD_TILE_BYTES is 0 without one)
    b200_es.ltile = (uint4*)(smem_gen + B200_STAGES * B200_STAGE_BYTES + B200_EPI_WARPS * B200_STAGING_TILES * B200_STAGING_BYTES +
                             ew * (unsigned int)B200_LOAD_TILE_BYTES);
    b200_es.lbar = bar_load + 8u * ew;
    b200_es.lph = 0u;
    b200_es.abort_flag = abort_flag;
    b200_es.status = status;
    B200_EPI_PROLOGUE
    unsigned int acc = 0, acc_phase = 0;
    // (batch, row, first column) of the part of a unit's tile that this thread works on
    auto b200_coords = [&](unsigned int u, unsigned int& tile, unsigned int& b0, unsigned int& b1, unsigned int& mt, unsigned int& nt) {
      tile = u % total_tiles;
      const unsigned int bidx = tile / tiles_per_batch;
      const unsigned int t = tile - bidx * tiles_per_batch;
      const unsigned int group = t / (B200_RASTER * shape.tiles_n);
      const unsigned int first_m = group * B200_RASTER;
      const unsigned int rows = min((unsigned int)B200_RASTER, shape.tiles_m - first_m);
      const unsigned int r = t - group * B200_RASTER * shape.tiles_n;
      mt = first_m + r % rows;
      nt = r / rows;
      b0 = bidx / shape.B1;
      b1 = bidx - b0 * shape.B1;
    };
    // operand tiles of the epilogue (bias, mask, residual rows ...): loaded for a tile's first chunk
    // before its accumulator is waited for -- by the previous tile's last chunk when there was one
    b200_in_tiles b200_tiles;
    bool b200_prefetched = false;
    for (unsigned int unit = worker; unit < total_units; unit += n_workers) {
      unsigned int tile, b200_b0, b200_b1, mt, nt;
      b200_coords(unit, tile, b200_b0, b200_b1, mt, nt);
      const unsigned int b200_m = mt * B200_BM + cta_rank * B200_CTA_M + quarter * 32u + lane;
      // one scratch slot per (tile, CTA, epilogue warp) for epilogues that end in a grid-wide sum
      const unsigned int b200_slot = (tile * (1u + B200_CTA_PAIR) + cta_rank) * B200_EPI_WARPS + ew;
      const unsigned int b200_nslots = total_tiles * (1u + B200_CTA_PAIR) * B200_EPI_WARPS;
      // this warp's share of the next tile, for the prefetch at the end of this one
      bool b200_nx_ok = false;
      unsigned int b200_nx_b0 = 0, b200_nx_b1 = 0, b200_nx_m = 0, b200_nx_n0 = 0;
      if (unit + n_workers < total_units) {
        unsigned int ntile, nmt, nnt;
        b200_coords(unit + n_workers, ntile, b200_nx_b0, b200_nx_b1, nmt, nnt);
        b200_nx_m = nmt * B200_BM + cta_rank * B200_CTA_M + quarter * 32u + lane;
        b200_nx_n0 = nnt * B200_BN + col_half * cols_per_warp;
        b200_nx_ok = b200_nx_n0 < shape.N;
      }
      B200_EPILOGUE_ROWS
      if (!b200_prefetched) {
        const unsigned int b200_pn0 = nt * B200_BN + col_half * cols_per_warp;
        if (b200_pn0 < shape.N) { B200_EPILOGUE_LOAD }
      }
      b200_prefetched = b200_nx_ok && (nt * B200_BN + col_half * cols_per_warp < shape.N);
      if (!b200_wait(bar_acc_full + 8u * acc, acc_phase, abort_flag, status, 4u)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (warp == 2 && lane == 0) { if (unit == worker) B200_TR(8); else if (unit == worker + n_workers) B200_TR(10); }
#ifdef B200_TRACE
      B200_TRE(3);   // waiting for the accumulator (and the operand prefetch before it)
#endif
      const unsigned int taddr = tmem_base + acc * B200_BN + ((quarter * 32u) << 16);
      // One register buffer: the epilogue issues the TMEM load of the next chunk as soon as it
      // has consumed the current one, so the load overlaps the epilogue's stores.  (The loop is
      // deliberately not unrolled: the generated epilogue can be thousands of instructions.)
      unsigned int b200_r[B200_EPI_CHUNK];
      const unsigned int col0 = col_half * cols_per_warp;
      if (nt * B200_BN + col0 < shape.N) b200_tmem_ld_chunk(taddr + col0, b200_r);
#pragma unroll 1
      for (unsigned int c = 0; c < cols_per_warp; c += B200_EPI_CHUNK) {
        const unsigned int col = col0 + c;
        const unsigned int b200_n0 = nt * B200_BN + col;
        if (b200_n0 >= shape.N) break;  // warp-uniform
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#ifdef B200_TRACE
        B200_TRE(4);
#endif
        const bool b200_has_next = (c + B200_EPI_CHUNK < cols_per_warp) && (b200_n0 + B200_EPI_CHUNK < shape.N);
        const unsigned int b200_next_taddr = taddr + col + B200_EPI_CHUNK;
        // every lane takes part: rows beyond M compute nothing but help move the chunk
        B200_EPILOGUE_ROW
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
#if B200_CTA_PAIR
      if (lane == 0) b200_mbar_arrive_cluster_relaxed(b200_map_to_cta(bar_acc_empty + 8u * acc, 0u));
#else
      if (lane == 0) b200_mbar_arrive_relaxed(bar_acc_empty + 8u * acc);
#endif
      if (warp == 2 && lane == 0) { if (unit == worker) B200_TR(9); else if (unit == worker + n_workers) B200_TR(11); }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
#ifdef B200_TRACE
      B200_TRE(5);   // release of the accumulator buffer
#endif
    }
    // the copy engine has read this warp's staging tiles before the CTA gives its shared memory back
    if (lane == 0) b200_tma_store_read_wait<0>();
#ifdef B200_TRACE
    b200_tre(0, true, status);
#endif
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag) {
    // let copies and MMAs already in flight land before the tensor memory is released
    const unsigned long long t0 = b200_now_ns();
    while (b200_now_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  b200_cluster_sync();   // neither CTA of a pair leaves while the other may still read its memory or signal its barriers
  if (threadIdx.x == 0) B200_TR(12);  // all roles done
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc." B200_CG ".sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned int)B200_TMEM_COLS)
                 : "memory");
  }
}

#endif  // B200_GEMM_SM100_CUH
