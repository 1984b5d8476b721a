// Building blocks shared by the tensor-core kernels for sm_100a (the contraction kernel and the
// fused attention kernel): mbarriers with bounded waits, TMA tile loads, shared-memory matrix
// descriptors, tcgen05.mma / commit, tensor-memory loads and stores.
//
// The including translation unit defines B200_ELEM_BYTES (operand element size) and may define
// B200_CTA_PAIR (1: two CTAs of a cluster work on one tile, cta_group::2).
#ifndef B200_TC_SM100_CUH
#define B200_TC_SM100_CUH

struct __align__(64) b200_tmap {
  unsigned long long opaque[16];
};


__device__ __forceinline__ unsigned int b200_smem_addr(const void* p) {
  return (unsigned int)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void b200_mbar_init(unsigned int bar, unsigned int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void b200_mbar_expect_tx(unsigned int bar, unsigned int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void b200_mbar_arrive(unsigned int bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ unsigned int b200_mbar_try(unsigned int bar, unsigned int parity) {
  unsigned int ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ unsigned long long b200_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#ifndef B200_WAIT_LIMIT_NS
#define B200_WAIT_LIMIT_NS 2000000000ull
#endif
// Bounded wait.  Returns false when the CTA is aborting or the limit passed (then it raises
// the abort flag and records `site` in the device status word).
__device__ __forceinline__ bool b200_wait(unsigned int bar, unsigned int parity, volatile unsigned int* abort_flag,
                                          unsigned int* status, unsigned int site) {
  if (b200_mbar_try(bar, parity)) return true;
  const unsigned long long t0 = b200_now_ns();
  for (unsigned int it = 1;; ++it) {
    if (b200_mbar_try(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag) return false;
      if (b200_now_ns() - t0 > B200_WAIT_LIMIT_NS) {
        *abort_flag = 1u;
        if (atomicCAS(status, 0u, 1u) == 0u) status[1] = site;
        __threadfence_system();
        return false;
      }
    }
  }
}

// B200_CTA_PAIR: two CTAs of a cluster (one TPC) work on one 256 x BN tile.  Each stages its own
// 128 rows of A and half of the BN columns of B; the even CTA (the leader) issues the
// cta_group::2 MMAs, which read both CTAs' shared memory and write each CTA's 128 accumulator rows
// into that CTA's tensor memory.  Per CTA the operand traffic into shared memory drops by a third.
#ifndef B200_CTA_PAIR
#define B200_CTA_PAIR 0
#endif
#if B200_CTA_PAIR
#define B200_CG "cta_group::2"
#else
#define B200_CG "cta_group::1"
#endif

__device__ __forceinline__ unsigned int b200_cta_rank() {
#if B200_CTA_PAIR
  unsigned int r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
#else
  return 0u;
#endif
}
// the shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ unsigned int b200_map_to_cta(unsigned int addr, unsigned int rank) {
#if B200_CTA_PAIR
  unsigned int r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
#else
  return addr;
#endif
}
__device__ __forceinline__ void b200_mbar_arrive_cluster(unsigned int cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Arrivals that order nothing in memory: the epilogue hands an accumulator buffer back after its
// tensor-memory loads have completed (tcgen05.wait::ld), and must not wait for the loads of its next
// operand tiles, which a releasing arrival would do.
__device__ __forceinline__ void b200_mbar_arrive_relaxed(unsigned int bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void b200_mbar_arrive_cluster_relaxed(unsigned int cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void b200_cluster_sync() {
#if B200_CTA_PAIR
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
#endif
}

__device__ __forceinline__ void b200_tma_load_4d(unsigned int dst, const b200_tmap* map, unsigned int bar, int c0, int c1,
                                                 int c2, int c3) {
  asm volatile(
#if B200_CTA_PAIR
      // the completion may be signalled on the peer CTA's barrier; each CTA loads only its own data
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
#else
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
#endif
      :
      : "r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Shared-memory matrix descriptor of tcgen05.mma for a 128-byte-swizzled tile.
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) descriptor version (1 on sm_100)
//   bits [61,64) swizzle mode: 2 = 16-byte chunks swizzled within 128 bytes over 8 rows;
//                1 = 32-byte chunks swizzled within 128 bytes over 4 rows, the only form the
//                tensor cores read an m/n-major operand of 32-bit elements in
__device__ __forceinline__ unsigned long long b200_smem_desc(unsigned int addr, unsigned int lbo_bytes,
                                                             unsigned int sbo_bytes, unsigned int swizzle_mode = 2u) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= (unsigned long long)swizzle_mode << 61;
  return d;
}
// m/n-major operands: 128-byte chunks of m/n, k rows 128 bytes apart in groups of 8 rows (1024
// bytes; 4 rows, 512 bytes, for 32-bit elements), chunks one TMA box apart
#if B200_ELEM_BYTES == 4
#define B200_MN_GROUP_BYTES 512u
#define B200_MN_SWIZZLE 1u
#else
#define B200_MN_GROUP_BYTES 1024u
#define B200_MN_SWIZZLE 2u
#endif

__device__ __forceinline__ void b200_umma(unsigned int tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                          unsigned int idesc, unsigned int accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
#if B200_ELEM_BYTES == 4
      "tcgen05.mma." B200_CG ".kind::tf32 [%0], %1, %2, %3, p;\n\t"
#else
      "tcgen05.mma." B200_CG ".kind::f16 [%0], %1, %2, %3, p;\n\t"
#endif
      "}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `bar` once the MMAs issued so far have retired; in pair mode on the barrier at the
// same offset in both CTAs.
__device__ __forceinline__ void b200_umma_commit(unsigned int bar) {
#if B200_CTA_PAIR
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"((unsigned short)3)
               : "memory");
#else
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
#endif
}
__device__ __forceinline__ void b200_tmem_ld32(unsigned int taddr, unsigned int* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void b200_tmem_ld16(unsigned int taddr, unsigned int* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void b200_tmem_st32(unsigned int taddr, const unsigned int* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// TMA store of a shared-memory tile (laid out as the tensor map's swizzle says) to global memory;
// elements outside the tensor are clipped by the copy engine.  One thread issues; the tile may be
// written again once b200_tma_store_read_wait says the copy has read it.
__device__ __forceinline__ void b200_tma_store_4d(const b200_tmap* map, unsigned int src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"((unsigned long long)map),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// the same without closing the group: several copies, then one b200_tma_commit
__device__ __forceinline__ void b200_tma_store_4d_nc(const b200_tmap* map, unsigned int src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"((unsigned long long)map),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void b200_tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until at most PENDING of this thread's copy groups still read shared memory
template <int PENDING>
__device__ __forceinline__ void b200_tma_store_read_wait() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory");
}

// Per-warp state of a contraction epilogue that the generated code shares with the kernel.
struct b200_epi_state {
  bool tma;                            // outputs leave as TMA stores, row operands arrive as TMA loads (the maps are valid)
  unsigned int nst;                    // != 0: this warp has copies in flight that read its staging tiles
  uint4* ltile;                        // tile that receives a row operand's chunk (32 rows, swizzled like a staging tile)
  unsigned int lbar;                   // its barrier (shared-memory address)
  unsigned int lph;                    // parity of the next completion to wait for
  volatile unsigned int* abort_flag;   // the CTA's abort flag and the device status word, for the bounded wait
  unsigned int* status;
};

#endif  // B200_TC_SM100_CUH
