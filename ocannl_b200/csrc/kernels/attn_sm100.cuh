// Fused attention stage for sm_100a: the chain
//     scores[b, s, h, t] = E1( sum_e q[b, s, h, e] * k[b, t, h, e], operands such as a mask[s, t] )
//     max[b, s, h]       = max_t scores            exp_vals = E3(scores, max)       (softmax pieces of
//     sum[b, s, h]       = sum_t exp_vals          weights  = E5(exp_vals, sum)      lib/nn_blocks.ml:137-143)
//     out[b, s, h, e]    = E6( sum_t weights[b, s, h, t] * v[b, t, h, e] )
// (multi_head_attention, lib/nn_blocks.ml:222-236) as ONE kernel.  A CTA takes 128 queries of one
// (batch, head): TMA brings the query rows, all B200_T keys and all values into shared memory,
// tcgen05.mma forms the 128 x T scores in tensor memory, the eight warps run the softmax passes on
// them -- a thread owns half of one row, the row's values go back to tensor memory between passes,
// the halves meet through shared memory -- the weights are written to shared memory in the
// operand layout of the tensor cores and a second tcgen05.mma forms the 128 x 64 output.  Scores,
// exponentials and weights are written to global memory only when the routine keeps those nodes
// (as TMA stores); max and sum likewise (their row pointers are non-null then).
//
// The translation unit that includes this text defines
//   B200_ATTN_NAME       kernel symbol
//   B200_T               keys per row: 64, 128 or 256        B200_E   head dimension: 64
//   B200_IDESC1/2        instruction descriptors of the two MMAs (128 x T x 16, 128 x E x 16)
//   B200_HALF            1: the weights are IEEE half, 0: bfloat16
//   B200_OUT_BYTES       element size of the output node (2 or 4)
//   B200_ATTN_NCOND      operands of the score expression that are only tested against zero (masks)
//   B200_ATTN_NTILES     operands of the score expression loaded a chunk at a time through the staging tile
//   B200_KEEP_SCORES / B200_KEEP_EXP / B200_KEEP_W   1: the routine keeps that node (it is written, by TMA stores)
//   B200_ATTN_PARAMS / B200_ATTN_ARGS    node pointers of the generated code
// and the generated functions b200_attn_score_chunk, b200_attn_exp_chunk, b200_attn_weight_chunk,
// b200_attn_out_chunk, b200_attn_row_max, b200_attn_row_sum, b200_attn_cond_rows and b200_attn_rows (see attn_match.cpp).
#ifndef B200_ATTN_SM100_CUH
#define B200_ATTN_SM100_CUH

struct b200_attn_shape {
  unsigned int S;          // queries per (batch, head)
  unsigned int B0, B1;     // batch extents, outer and inner
  unsigned int tiles_s;    // ceil(S / 128)
};

#define B200_ATTN_THREADS 256
#define B200_Q_BYTES (128 * B200_E * 2)
#define B200_K_BYTES (B200_T * B200_E * 2)
#define B200_V_BYTES (B200_T * B200_E * 2)
#define B200_P_BYTES (128 * B200_T * 2)
// region A holds, one after the other in time: the query and key tiles; the warps' staging tiles
// of the first two passes; the weights
#define B200_STAGE_WARP_BYTES 4096
#define B200_RA0 (B200_Q_BYTES + B200_K_BYTES)
#define B200_RA1 (B200_RA0 > B200_P_BYTES ? B200_RA0 : B200_P_BYTES)
#define B200_REGION_A (B200_RA1 > 8 * B200_STAGE_WARP_BYTES ? B200_RA1 : 8 * B200_STAGE_WARP_BYTES)
// staging tiles per warp for the TMA stores of the first two passes (region A is free of operands then)
#define B200_STAGE_BUFS ((B200_REGION_A >= 16 * B200_STAGE_WARP_BYTES && B200_ATTN_NTILES == 0) ? 2 : 1)
#define B200_ATTN_TMEM_COLS (B200_T < 64 ? 64 : B200_T)
#define B200_HALF_COLS (B200_T / 2)

// Stores a chunk of 32 rows x (4 * WORDS) bytes that the warp holds one row per lane.  Storing from
// registers would touch 32 lines per instruction, so the chunk is transposed through a swizzled
// staging tile and every instruction writes whole row segments.  `row_ptr` is the address of the
// chunk's first byte in this lane's row (0: the row is not written).
template <int WORDS>
__device__ __forceinline__ void b200_attn_store_chunk(uint4* stage, const unsigned int* w, unsigned long long row_ptr, unsigned int lane) {
  constexpr int G = WORDS / 4;                         // 16-byte groups per row
  constexpr unsigned int RPK = G >= 8 ? 1u : 8u / G;   // rows that share one 128-byte line of the tile
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const unsigned int key = (lane / RPK) % (G >= 8 ? 8u : (unsigned int)G);
    stage[lane * G + ((unsigned int)g ^ key)] = make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
  }
  __syncwarp();
#pragma unroll
  for (int it = 0; it < G; ++it) {
    const unsigned int r = it * (32 / G) + lane / G, c = lane % G;
    const unsigned long long dst = __shfl_sync(0xffffffffu, row_ptr, r);
    const unsigned int key = (r / RPK) % (G >= 8 ? 8u : (unsigned int)G);
    const uint4 q = stage[r * G + (c ^ key)];
    if (dst) *(uint4*)(dst + 16ull * c) = q;
  }
  __syncwarp();
}

// A chunk of 32 rows x 32 single-precision columns that the warp holds one row per lane goes to
// global memory as ONE TMA store: the lanes write their rows into a 4 KB tile in the 128-byte
// swizzle the tensor map describes, lane 0 issues the copy and moves on; rows beyond the node's
// extent are clipped by the copy engine.  The tile may be written again once the copy has read it
// (b200_attn_tile_free).
__device__ __forceinline__ void b200_attn_tma_store_chunk(unsigned char* tile, const unsigned int* u, const b200_tmap* map, int t0, int s0,
                                                          int b1, int b0, unsigned int lane) {
  uint4* st = (uint4*)tile;
#pragma unroll
  for (unsigned int g = 0; g < 8u; ++g) st[lane * 8u + (g ^ (lane & 7u))] = make_uint4(u[4 * g], u[4 * g + 1], u[4 * g + 2], u[4 * g + 3]);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (lane == 0) b200_tma_store_4d(map, b200_smem_addr(tile), t0, s0, b1, b0);
}

// The reverse: loads a chunk of 32 rows x (4 * WORDS) bytes with whole-row-segment accesses and
// hands every lane its own row.  Rows whose pointer is 0 read as zero bits.
template <int WORDS>
__device__ __forceinline__ void b200_attn_load_chunk(uint4* stage, unsigned int* w, unsigned long long row_ptr, unsigned int lane) {
  constexpr int G = WORDS / 4;
  constexpr unsigned int RPK = G >= 8 ? 1u : 8u / G;
#pragma unroll
  for (int it = 0; it < G; ++it) {
    const unsigned int r = it * (32 / G) + lane / G, c = lane % G;
    const unsigned long long src = __shfl_sync(0xffffffffu, row_ptr, r);
    const unsigned int key = (r / RPK) % (G >= 8 ? 8u : (unsigned int)G);
    uint4 q = make_uint4(0u, 0u, 0u, 0u);
    if (src) q = *(const uint4*)(src + 16ull * c);
    stage[r * G + (c ^ key)] = q;
  }
  __syncwarp();
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const unsigned int key = (lane / RPK) % (G >= 8 ? 8u : (unsigned int)G);
    const uint4 q = stage[lane * G + ((unsigned int)g ^ key)];
    w[4 * g] = q.x; w[4 * g + 1] = q.y; w[4 * g + 2] = q.z; w[4 * g + 3] = q.w;
  }
  __syncwarp();
}

// Developer aid: with -DB200_TRACE, thread 0 of one CTA (B200_TRACE_CTA, default 0) records nanoseconds
// since its start at a few points into words 40.. of the device status buffer.
#ifdef B200_TRACE
#ifndef B200_TRACE_CTA
#define B200_TRACE_CTA 0
#endif
#define B200_ATR(slot) do { if (blockIdx.x == B200_TRACE_CTA && threadIdx.x == 0) status[40 + slot] = (unsigned int)(b200_now_ns() - b200_t0); } while (0)
#else
#define B200_ATR(slot) do { } while (0)
#endif

// what the generated code needs to know about this thread's row
struct b200_attn_row {
  unsigned int b0, b1, s;   // batch indices and query position
  bool ok;                  // s < S
  unsigned int lane;
  uint4* stage;             // this warp's staging tile
};

// generated per routine (defined after this text)
__device__ __forceinline__ float b200_attn_max_init();
__device__ __forceinline__ void b200_attn_rows(const b200_attn_row& row, unsigned long long& p_max, unsigned long long& p_sum,
                                               unsigned long long& p_out B200_ATTN_PARAMS);
__device__ __forceinline__ void b200_attn_cond_rows(const b200_attn_row& row, unsigned long long* p B200_ATTN_PARAMS);
__device__ __forceinline__ void b200_attn_score_chunk(const b200_attn_row& row, unsigned int t0, const unsigned int* acc, float* x,
                                                      const unsigned int* cw B200_ATTN_PARAMS);
__device__ __forceinline__ float b200_attn_row_max(const b200_attn_row& row, float reduced B200_ATTN_PARAMS);
__device__ __forceinline__ void b200_attn_exp_chunk(const b200_attn_row& row, unsigned int t0, float* x, float mx B200_ATTN_PARAMS);
__device__ __forceinline__ float b200_attn_row_sum(const b200_attn_row& row, float reduced B200_ATTN_PARAMS);
__device__ __forceinline__ void b200_attn_weight_chunk(const b200_attn_row& row, unsigned int t0, const float* e, float sum, unsigned int* w B200_ATTN_PARAMS);
__device__ __forceinline__ void b200_attn_out_chunk(const b200_attn_row& row, unsigned int e0, const unsigned int* acc, unsigned int* w B200_ATTN_PARAMS);

extern "C" __global__ void __launch_bounds__(B200_ATTN_THREADS, 2)
B200_ATTN_NAME(const __grid_constant__ b200_tmap map_q, const __grid_constant__ b200_tmap map_k,
               const __grid_constant__ b200_tmap map_v, const __grid_constant__ b200_tmap map_scores,
               const __grid_constant__ b200_tmap map_exp, const __grid_constant__ b200_tmap map_w, const b200_attn_shape shape,
               unsigned int* status B200_ATTN_PARAMS) {
  extern __shared__ unsigned char b200_dyn_smem[];
  const unsigned int smem_base = (b200_smem_addr(b200_dyn_smem) + 1023u) & ~1023u;
  unsigned char* smem_gen = b200_dyn_smem + (smem_base - b200_smem_addr(b200_dyn_smem));
  const unsigned int q_at = smem_base, k_at = smem_base + B200_Q_BYTES, p_at = smem_base;
  const unsigned int v_at = smem_base + B200_REGION_A;
  unsigned char* after = smem_gen + B200_REGION_A + B200_V_BYTES;
  float* red = (float*)after;                                         // [2][128]: the column halves of a row meet here
  unsigned long long* bars = (unsigned long long*)(after + 1024);
  const unsigned int bar_qk = b200_smem_addr(bars), bar_v = bar_qk + 8u, bar_s = bar_qk + 16u, bar_o = bar_qk + 24u;
  volatile unsigned int* tmem_slot = (volatile unsigned int*)(bars + 4);
  volatile unsigned int* abort_flag = tmem_slot + 1;

  asm volatile("griddepcontrol.launch_dependents;");
  const unsigned int warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const unsigned int quarter = warp & 3u, half = warp >> 2;
#ifdef B200_TRACE
  const unsigned long long b200_t0 = b200_now_ns();
#endif

  if (threadIdx.x == 32) {
#if B200_KEEP_SCORES
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_scores) : "memory");
#endif
#if B200_KEEP_EXP
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_exp) : "memory");
#endif
#if B200_KEEP_W
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_w) : "memory");
#endif
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_v) : "memory");
  }
  if (threadIdx.x == 0) {
    b200_mbar_init(bar_qk, 1);
    b200_mbar_init(bar_v, 1);
    b200_mbar_init(bar_s, 1);
    b200_mbar_init(bar_o, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(b200_smem_addr((const void*)tmem_slot)),
                 "r"((unsigned int)B200_ATTN_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned int tmem_base = *tmem_slot;
  B200_ATR(0);   // set-up done

  // this CTA's (batch, head, query tile); neighbouring CTAs share keys and values
  const unsigned int st = blockIdx.x % shape.tiles_s;
  const unsigned int bh = blockIdx.x / shape.tiles_s;
  const unsigned int b0 = bh / shape.B1, b1 = bh - b0 * shape.B1;
  const unsigned int s0 = st * 128u;

  if (threadIdx.x == 0) {
    b200_mbar_expect_tx(bar_qk, B200_Q_BYTES + B200_K_BYTES);
    b200_tma_load_4d(q_at, &map_q, bar_qk, 0, (int)s0, (int)b1, (int)b0);
    b200_tma_load_4d(k_at, &map_k, bar_qk, 0, 0, (int)b1, (int)b0);
    b200_mbar_expect_tx(bar_v, B200_V_BYTES);
    b200_tma_load_4d(v_at, &map_v, bar_v, 0, 0, (int)b1, (int)b0);
    // scores = q . k^T: both operands k-major, rows of 128 bytes, 8-row groups 1024 bytes apart
    if (b200_wait(bar_qk, 0u, abort_flag, status, 11u)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      B200_ATR(1);   // queries and keys landed
      const unsigned long long dq = b200_smem_desc(q_at, 16u, 1024u), dk = b200_smem_desc(k_at, 16u, 1024u);
#pragma unroll
      for (unsigned int ks = 0; ks < B200_E / 16; ++ks)
        b200_umma(tmem_base, dq + (unsigned long long)((ks * 32u) >> 4), dk + (unsigned long long)((ks * 32u) >> 4),
                  (unsigned int)B200_IDESC1, ks != 0u ? 1u : 0u);
      b200_umma_commit(bar_s);
    }
  }
  __syncwarp();

  b200_attn_row row;
  row.b0 = b0; row.b1 = b1;
  row.s = s0 + quarter * 32u + lane;
  row.ok = row.s < shape.S;
  row.lane = lane;
  // this warp's staging tiles (B200_STAGE_BUFS of 4 KB each, 1024-byte aligned)
  unsigned char* const my_tiles = smem_gen + warp * (B200_STAGE_BUFS * B200_STAGE_WARP_BYTES);
  row.stage = (uint4*)my_tiles;
  unsigned int n_stores = 0;   // chunks this warp has handed to the copy engine
  (void)n_stores;
  const unsigned int r_in_tile = quarter * 32u + lane;
  const unsigned int col0 = half * B200_HALF_COLS;
  const unsigned int taddr = tmem_base + ((quarter * 32u) << 16);
  // row pointers of the per-row nodes this routine keeps and of the output (byte address of this thread's
  // row; 0: not written); scores, exponentials and weights leave through their tensor maps
  unsigned long long p_max, p_sum, p_out;
  b200_attn_rows(row, p_max, p_sum, p_out B200_ATTN_ARGS);

  // Operands of the score expression that are only tested against zero (masks) arrive packed to one
  // bit per element: this thread's half row is B200_HALF_COLS / 32 words, fetched while the queries
  // and keys are still on their way.  cond[4 * i + k] bit j = column 32 * k + j of the half.
#if B200_ATTN_NCOND > 0
  unsigned int cond[4 * B200_ATTN_NCOND];
  {
    unsigned long long cp[B200_ATTN_NCOND];
    b200_attn_cond_rows(row, cp B200_ATTN_ARGS);
#pragma unroll
    for (int i = 0; i < B200_ATTN_NCOND; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        cond[4 * i + k] = (cp[i] && k < (int)(B200_HALF_COLS / 32)) ? ((const unsigned int*)(cp[i] + col0 / 8u))[k] : 0u;
    }
  }
#endif

  bool live = b200_wait(bar_s, 0u, abort_flag, status, 12u);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  // One chunk of 32 columns at a time; the tensor-memory load of the next chunk is issued as soon as
  // the current one has been consumed, so that it overlaps the arithmetic and the stores.
  unsigned int acc[32];
  float x[32];
  B200_ATR(2);   // scores in tensor memory
  if (live) {
    // ---- pass 1: scores, running max
    // (four running values each for the maximum and the sum: neighbouring elements do not wait for one another)
    float mx4[4] = {b200_attn_max_init(), b200_attn_max_init(), b200_attn_max_init(), b200_attn_max_init()};
    b200_tmem_ld32(taddr + col0, acc);
#pragma unroll 1
    for (unsigned int c = 0; c < B200_HALF_COLS; c += 32u) {
      const unsigned int t0 = col0 + c;
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#if B200_ATTN_NTILES > 0 && B200_KEEP_SCORES
      // the operand tiles of this chunk pass through the staging tile the previous chunk's store reads
      if (lane == 0) b200_tma_store_read_wait<0>();
      __syncwarp();
#endif
      unsigned int cw[B200_ATTN_NCOND > 0 ? B200_ATTN_NCOND : 1];
#if B200_ATTN_NCOND > 0
#pragma unroll
      for (int i = 0; i < B200_ATTN_NCOND; ++i)   // this chunk's word (selects: the word index is not a compile-time constant)
        cw[i] = c == 0u ? cond[4 * i] : c == 32u ? cond[4 * i + 1] : c == 64u ? cond[4 * i + 2] : cond[4 * i + 3];
#else
      cw[0] = 0u;
#endif
      b200_attn_score_chunk(row, t0, acc, x, cw B200_ATTN_ARGS);
      if (c + 32u < B200_HALF_COLS) b200_tmem_ld32(taddr + t0 + 32u, acc);
      unsigned int u[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) { mx4[j & 3] = fmaxf(mx4[j & 3], x[j]); u[j] = __float_as_uint(x[j]); }
      b200_tmem_st32(taddr + t0, u);
#if B200_KEEP_SCORES
      if (n_stores >= B200_STAGE_BUFS) {
        if (lane == 0) b200_tma_store_read_wait<B200_STAGE_BUFS - 1>();
        __syncwarp();
      }
      b200_attn_tma_store_chunk(my_tiles + (n_stores % B200_STAGE_BUFS) * B200_STAGE_WARP_BYTES, u, &map_scores, (int)t0,
                                (int)(s0 + quarter * 32u), (int)b1, (int)b0, lane);
      ++n_stores;
#endif
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    red[half * 128u + r_in_tile] = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
  }
  B200_ATR(3);   // pass 1 done
  __syncthreads();
  float mx_row = 0.f, sum_row = 0.f;
  if (live) {
    mx_row = b200_attn_row_max(row, fmaxf(red[r_in_tile], red[128u + r_in_tile]) B200_ATTN_ARGS);
    if (half == 0u && p_max) *(float*)p_max = mx_row;
  }
  __syncthreads();   // `red` is reused for the sums
  if (live) {
    // ---- pass 2: exponentials, running sum
    float sum4[4] = {0.f, 0.f, 0.f, 0.f};
    b200_tmem_ld32(taddr + col0, acc);
#pragma unroll 1
    for (unsigned int c = 0; c < B200_HALF_COLS; c += 32u) {
      const unsigned int t0 = col0 + c;
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(acc[j]);
      if (c + 32u < B200_HALF_COLS) b200_tmem_ld32(taddr + t0 + 32u, acc);
      b200_attn_exp_chunk(row, t0, x, mx_row B200_ATTN_ARGS);
      unsigned int u[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) { sum4[j & 3] += x[j]; u[j] = __float_as_uint(x[j]); }
      b200_tmem_st32(taddr + t0, u);
#if B200_KEEP_EXP
      if (n_stores >= B200_STAGE_BUFS) {
        if (lane == 0) b200_tma_store_read_wait<B200_STAGE_BUFS - 1>();
        __syncwarp();
      }
      b200_attn_tma_store_chunk(my_tiles + (n_stores % B200_STAGE_BUFS) * B200_STAGE_WARP_BYTES, u, &map_exp, (int)t0,
                                (int)(s0 + quarter * 32u), (int)b1, (int)b0, lane);
      ++n_stores;
#endif
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    red[half * 128u + r_in_tile] = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
  }
#if B200_KEEP_SCORES || B200_KEEP_EXP
  if (lane == 0) b200_tma_store_read_wait<0>();   // the copy engine has read every staging tile: region A may change hands
#endif
  B200_ATR(4);   // pass 2 done
  __syncthreads();   // also: every warp is done with its staging tile, region A may take the weights
  if (live) {
    sum_row = b200_attn_row_sum(row, red[r_in_tile] + red[128u + r_in_tile] B200_ATTN_ARGS);
    if (half == 0u && p_sum) *(float*)p_sum = sum_row;
    // ---- pass 3: weights, into shared memory as the k-major A operand of the second MMA: blocks of
    //      64 keys, a row of a block is 128 bytes whose 16-byte pieces are xor-swizzled with (row % 8)
    b200_tmem_ld32(taddr + col0, acc);
#pragma unroll 1
    for (unsigned int c = 0; c < B200_HALF_COLS; c += 32u) {
      const unsigned int t0 = col0 + c;
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(acc[j]);
      if (c + 32u < B200_HALF_COLS) b200_tmem_ld32(taddr + t0 + 32u, acc);
      unsigned int w[16];
      b200_attn_weight_chunk(row, t0, x, sum_row, w B200_ATTN_ARGS);
      unsigned char* prow = smem_gen + (t0 >> 6) * (128u * 128u) + r_in_tile * 128u;
      const unsigned int piece0 = (t0 & 63u) >> 3;   // first 16-byte piece of this chunk in the row: 0 or 4
#pragma unroll
      for (unsigned int g = 0; g < 4; ++g)
        *(uint4*)(prow + (((piece0 + g) ^ (r_in_tile & 7u)) << 4)) = make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
    }
    // the tensor cores read shared memory through the async proxy
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  B200_ATR(5);   // pass 3 done
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && live) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (b200_wait(bar_v, 0u, abort_flag, status, 13u)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // out = weights . v: A k-major (blocks of 64 keys, 16 KB apart), B n-major (rows of 64 head
      // dimensions = 128 bytes per key, 8-key groups 1024 bytes apart)
      const unsigned long long dp = b200_smem_desc(p_at, 16u, 1024u);
      const unsigned long long dv = b200_smem_desc(v_at, 64u * 64u * 2u, 1024u);
#pragma unroll
      for (unsigned int ks = 0; ks < B200_T / 16; ++ks) {
        const unsigned int a_off = (ks >> 2) * (128u * 128u) + (ks & 3u) * 32u;
        const unsigned int b_off = ks * 16u * 128u;
        b200_umma(tmem_base, dp + (unsigned long long)(a_off >> 4), dv + (unsigned long long)(b_off >> 4), (unsigned int)B200_IDESC2,
                  ks != 0u ? 1u : 0u);
      }
      b200_umma_commit(bar_o);
    }
    B200_ATR(6);   // second MMA issued
#if B200_KEEP_W
    // the weights go to global memory straight from the operand tile, one TMA store per block of
    // 64 keys, while the tensor cores read the same tile
#pragma unroll
    for (unsigned int kb = 0; kb < B200_T / 64; ++kb) b200_tma_store_4d(&map_w, p_at + kb * (128u * 128u), (int)(kb * 64u), (int)s0, (int)b1, (int)b0);
    b200_tma_store_read_wait<0>();
#endif
  }
  __syncwarp();
  B200_ATR(7);   // weights copied out
  live = live && b200_wait(bar_o, 0u, abort_flag, status, 14u);
  B200_ATR(8);   // output accumulators ready
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncthreads();   // nobody reads the weights in region A any more: it takes the staging tiles again
  if (live) {
    // ---- output: 32 of the 64 head dimensions per thread
    const unsigned int e0 = half * 32u;
    b200_tmem_ld32(taddr + e0, acc);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    unsigned int w[32 * B200_OUT_BYTES / 4];
    b200_attn_out_chunk(row, e0, acc, w B200_ATTN_ARGS);
    b200_attn_store_chunk<32 * B200_OUT_BYTES / 4>(row.stage, w, p_out ? p_out + (unsigned long long)B200_OUT_BYTES * e0 : 0ull, lane);
  }

  B200_ATR(9);   // output stored
  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = b200_now_ns();
    while (b200_now_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned int)B200_ATTN_TMEM_COLS) : "memory");
  }
}

#endif  // B200_ATTN_SM100_CUH
