// Non-causal attention of a query chunk over a key/value window, bf16 in / bf16 out, fp32
// softmax, on tcgen05 tensor cores (kind::f16) with the score and output accumulators in tensor
// memory.  head_dim = 128.
//
//   O[q, h, :] = softmax_k( Q[q, h, :] . K[k, h, :] * scale ) V[k, h, :]
//
// One CTA per (256-query tile, head), 10 warps.  The tile is processed as two independent
// 128-query halves that share the K/V tiles; each half has its own score / output accumulator
// (S_h, O_h: 4 x 128 columns = the whole tensor memory) and its own softmax warpgroup, so that
// the tensor pipe works on one half while the other half is in its softmax:
//   warp 0     TMA producer: both Q halves once, then K and V tiles of 128 keys (two 64-channel
//              halves each, 128-byte swizzle), two stages.
//   warp 1     MMA issuer / TMEM owner.  S_h = Q_h K_j^T (8 MMAs, K = 16 channels, operands K-major
//              in shared memory); O_h += P_h V_j (8 MMAs, K = 16 keys; P read from tensor memory
//              where it overwrote S_h, V MN-major in shared memory).  Issue order per key tile:
//              PV_a(j), S_a(j+1), PV_b(j), S_b(j+1).
//   warps 2-5  softmax of half a, warps 6-9 softmax of half b: thread = query row.  Reads S with
//              tcgen05.ld, keeps the running row maximum and sum, writes P as packed bf16 over the
//              first 64 columns of the score buffer (tcgen05.st).  The output accumulator is
//              rescaled lazily: only when a row maximum grows by more than 2^8 is O multiplied by
//              exp2(m_old - m_new), so in steady state O is touched only by the tensor pipe.
//              After the last tile the same warps normalise O and store it through swizzled
//              shared memory (the Q tile's buffer) with TMA.
// All mbarrier waits are bounded (sm100.cuh).
//
// NVFP4 key/value cache (attention_kernel<true>, llnv_attention_nvfp4kv).  The window is a list of
// segments: cached NVFP4 blocks (E2M1 codes, E4M3 scale per 16 channels, one fp32 amax per block,
// rows ordered token-major / head-minor) followed by the current chunk in bf16.  The cached part is
// never materialised in global memory: four more warps (12-15) decode it inside the load stage.
// The TMA producer loads the 128 x 64-byte code tile of the stage's next key tile (one box per cache
// block the tile touches, at most two) into the tail of the K / V stage itself, which is free at
// that point; decode thread i owns key row i: it reads the row's 64 code bytes from there and its 8
// scale bytes from global memory (prefetched one tile ahead) and writes the bf16 row over the stage
// in the 128-byte-swizzled layout the MMAs read -- the same bytes a TMA load of the dequantized
// window would have put there, so the result equals dequantize-then-attention bit for bit.  (Row
// loads issued by the decode threads themselves -- 64 bytes per thread, every lane in another cache
// line -- kept the load/store unit busy for longer than the decode itself; one TMA box per tile
// does not touch it.)  The value of a code is that of the standalone dequantize kernel,
//     bf16( (e2m1 * e4m3) * (amax * fp32(1 / (6 * 256))) ),
// which for one cache block depends only on (scale byte, code): when a tile first touches a cache
// block the decode warps compute, with exactly that arithmetic, the eight bf16 magnitudes of each of
// the 128 scale bytes into a 2 KiB shared-memory table (byte-split for prmt), and a row is then
// decoded with byte permutes alone: per 16 channels one 16-byte table read, per 8 channels four
// lookups, the sign bits, four interleaves.  No conversion or multiply runs per element, so the
// decode stays off the special-function pipe the softmax's exp2 lives on.  A tile that holds the
// last cached keys and the first keys of the current chunk is also built by these warps (they copy
// the bf16 rows); tiles that lie entirely in the current chunk come from TMA as before.
// Warp roles of this instantiation (16 warps): 0 = Q and K loads (code tiles or bf16 tiles), 1 = MMA issuer, 2 = V loads,
// 3 idle, 4-7 / 8-11 = softmax of half a / b, 12-15 = decode.  The register file is re-divided at the top of each role's
// branch (setmaxnreg): load / MMA warpgroup 56, decode warpgroup 104, softmax warpgroups 176.
//
// Work split.  blockIdx.z = key split: with nsplit > 1 every (query tile, head) item is cut into nsplit equal ranges of key
// tiles, each CTA writes unnormalised fp32 partials and (m, l), and attention_combine_kernel merges them (head shards with
// too few items to fill the device).  Tail balancing (tail_cut > 0) cuts only the items of the last partial wave, once, into a
// long and a short CTA, so that the short ones fill the SMs the long ones leave free (see tail_cut_for).
#include <cuda.h>
#include <cuda_fp4.h>

#include "common.cuh"
#include "sm100.cuh"

namespace llnv {
namespace {

using namespace sm100;

constexpr int kD = 128;            // head dim
constexpr int kBQ = 256;           // queries per CTA (two halves of 128)
constexpr int kHQ = 128;           // queries per half
constexpr int kBK = 128;           // keys per tile
constexpr int kStages = 2;
constexpr uint32_t kHalfBytes = 128 * 128;        // 128 rows x 64 bf16
constexpr uint32_t kTileBytes = 2 * kHalfBytes;   // 32 KiB
constexpr uint32_t kQOff = 0;
constexpr uint32_t kKOff = 2 * kTileBytes;
constexpr uint32_t kVOff = kKOff + kStages * kTileBytes;
constexpr uint32_t kBarOff = kVOff + kStages * kTileBytes;
constexpr uint32_t kSmemBytes = kBarOff + 1024;
// NVFP4 window: decode tables behind the barriers, kTabSlots cache blocks x (K, V) x 128 scale bytes x 16 bytes
constexpr int kTabSlots = 2;                      // a tile of 128 keys touches at most two cache blocks (blocks hold >= 128 tokens)
constexpr uint32_t kCodeBytes = 128 * 64;         // code tile of one cache block: 128 key rows x 64 bytes, 64-byte swizzle
constexpr uint32_t kCodeOff = kTileBytes - 2 * kCodeBytes;      // two code tiles in the tail of the stage they expand into
constexpr uint32_t kTabOff = kBarOff + 1024;
constexpr uint32_t kTabBytes = kTabSlots * 2 * 128 * 16;
constexpr uint32_t kSmemBytesFused = kTabOff + kTabBytes;
static_assert(kSmemBytesFused <= 232448, "more shared memory than one CTA may use");
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSCol = 0, kOCol = 256;      // S_h at kSCol + 128 h, O_h at kOCol + 128 h
constexpr int kThreads = 320;            // bf16 window: load, MMA, 2 x 4 softmax warps
constexpr int kThreadsFused = 512;       // NVFP4 window: four warpgroups (load + MMA, softmax a, softmax b, decode)
constexpr int kMaxKvBlocks = 16;

// Device pointers of the cached blocks of one layer (oldest first), passed as launch parameters.
struct KvTable {
  const uint8_t* k_sf[kMaxKvBlocks];
  const float* k_amax[kMaxKvBlocks];
  const uint8_t* v_sf[kMaxKvBlocks];
  const float* v_amax[kMaxKvBlocks];
  // codes of block b viewed as [block_tokens, heads * 64 bytes]: box = 128 tokens x the 64 bytes of one head
  CUtensorMap k_codes[kMaxKvBlocks];
  CUtensorMap v_codes[kMaxKvBlocks];
};

struct AttnParams {
  int64_t Lq, Lk;
  int heads;
  float scale_log2;            // scale * log2(e)
  unsigned int* status;
  // key splits: CTA z of a (query tile, head) handles a contiguous range of the key tiles and,
  // when there is more than one split, writes its unnormalised output and (m, l) to the workspace
  // tail balancing (tail_cut > 0, nsplit == 1, grid z = 2): (query tile, head) items are numbered in launch order
  // (tile + tiles * head); items below tail_first run whole in their z = 0 CTA, the others are cut at key tile
  // tail_cut into a z = 0 CTA and a shorter z = 1 CTA, both writing partial results
  int nsplit, tail_first, tail_cut;
  float* part_o;               // [nsplit][Lq][heads][128] fp32
  float* part_ml;              // [nsplit][Lq][heads][2]   fp32: exponent offset m (raw score units), sum l
  float* out_amax;             // optional: max |out| over all written elements (zeroed by the host before the launch)
  // NVFP4 window (attention_kernel<true>): the first n_cached keys live in cache blocks of block_tokens
  // tokens each, the remaining Lk - n_cached keys are the bf16 tensors the K / V tensor maps describe
  int64_t n_cached;
  int block_tokens;
  float inv_denom;             // fp32(1 / (e2m1_max * e4m3_max))
  const uint16_t* k_cur;       // current chunk, bf16 [Lk - n_cached, heads * 128]: rows of the tile shared with the cache
  const uint16_t* v_cur;
  int64_t ldk, ldv;
};

template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// What a decode thread keeps of its key row between the prefetch and the decode.
struct RowInfo {
  uint32_t ksf[2], vsf[2];      // kind 0: the row's 8 K and 8 V scale bytes
  int kind;                     // 0 = cache block, 1 = current chunk, 2 = beyond the window
  int where;                    // kind 0: row inside the staged code tiles (128.. = second tile) | table slot << 8;
                                // kind 1: row of the current chunk
};

// Decode table of one (cache block, scale byte): the bf16 magnitudes of the eight E2M1 magnitudes
// {0, .5, 1, 1.5, 2, 3, 4, 6} under that scale, computed as decode16<LLNV_DEQ_FUSED> of the standalone
// dequantize kernel computes them, stored byte-split: x = low bytes of magnitudes 0..3, y = low bytes of
// 4..7, z / w = the high bytes.
__device__ __forceinline__ uint4 decode_table_entry(uint32_t scale_byte, float g) {
  const float s = e4m3_to_float(scale_byte);
  const float mags[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  uint32_t pk[4];
#pragma unroll
  for (int m = 0; m < 4; ++m)
    pk[m] = pack_bf16x2(__fmul_rn(__fmul_rn(mags[2 * m], s), g), __fmul_rn(__fmul_rn(mags[2 * m + 1], s), g));
  uint4 t;
  t.x = __byte_perm(pk[0], pk[1], 0x6420);
  t.y = __byte_perm(pk[2], pk[3], 0x6420);
  t.z = __byte_perm(pk[0], pk[1], 0x7531);
  t.w = __byte_perm(pk[2], pk[3], 0x7531);
  return t;
}

// 8 codes (one word) -> 8 bf16 (16 bytes) with the table entry `t` of the codes' scale byte: four byte lookups
// (low / high bytes of codes 0..3 and 4..7), the sign bits, four interleaves.
__device__ __forceinline__ uint4 decode_word(uint32_t w, const uint4& t) {
  const uint32_t sel = w & 0x77777777u;             // magnitude indices of codes 0..3 (low half) and 4..7
  const uint32_t selb = sel >> 16;
  const uint32_t w4 = w << 4;                       // bit 7 of byte k: sign of code 2k (of w: sign of code 2k+1)
  const uint32_t lo_a = __byte_perm(t.x, t.y, sel), lo_b = __byte_perm(t.x, t.y, selb);
  uint32_t hi_a = __byte_perm(t.z, t.w, sel), hi_b = __byte_perm(t.z, t.w, selb);
  hi_a |= __byte_perm(w4, w, 0x5140) & 0x80808080u;
  hi_b |= __byte_perm(w4, w, 0x7362) & 0x80808080u;
  return make_uint4(__byte_perm(lo_a, hi_a, 0x5140), __byte_perm(lo_a, hi_a, 0x7362), __byte_perm(lo_b, hi_b, 0x5140),
                    __byte_perm(lo_b, hi_b, 0x7362));
}

// Decode a cached row (code words w[0..15], scale bytes sf0 | sf1) into row i of a K / V stage: two halves of 64
// channels, rows of 128 bytes, 16-byte chunks XOR-swizzled with the row index as a TMA load with the 128-byte
// swizzle writes them.  `tab` is the row's block's table (128 entries of 16 bytes) in shared memory.  The loop
// over the four 32-channel groups stays rolled (the words rotate through w[0..3]): unrolled, this code and the
// softmax's together overflow the instruction cache.
__device__ __forceinline__ void decode_row(uint32_t (&w)[16], uint32_t sf0, uint32_t sf1, const uint8_t* tab, uint8_t* stage, int i) {
  uint8_t* dst = stage + i * 128;
  const int x = i & 7;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {                       // 32 channels: two scale bytes, four 16-byte chunks
    const uint32_t sfw = (c & 2 ? sf1 : sf0) >> (16 * (c & 1));
    // table entries of the two scale bytes (bit 7 of a UE4M3 scale is never set): byte * 16
    const uint4 t0 = *reinterpret_cast<const uint4*>(tab + ((sfw << 4) & 0x7F0u));
    const uint4 t1 = *reinterpret_cast<const uint4*>(tab + ((sfw >> 4) & 0x7F0u));
    uint8_t* half = dst + (c >> 1) * kHalfBytes;
    const int k0 = (c & 1) * 4;                       // first chunk of the group inside its half
    *reinterpret_cast<uint4*>(half + (((k0 + 0) ^ x) << 4)) = decode_word(w[0], t0);
    *reinterpret_cast<uint4*>(half + (((k0 + 1) ^ x) << 4)) = decode_word(w[1], t0);
    *reinterpret_cast<uint4*>(half + (((k0 + 2) ^ x) << 4)) = decode_word(w[2], t1);
    *reinterpret_cast<uint4*>(half + (((k0 + 3) ^ x) << 4)) = decode_word(w[3], t1);
#pragma unroll
    for (int k = 0; k < 12; ++k) w[k] = w[k + 4];
  }
}

// Row i of a stage from 128 bf16 values in global memory (src == nullptr: zeros).
__device__ __forceinline__ void copy_row(const uint16_t* src, uint8_t* stage, int i) {
#pragma unroll 4
  for (int chunk = 0; chunk < 16; ++chunk) {
    const uint4 v = src ? __ldg(reinterpret_cast<const uint4*>(src) + chunk) : make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(stage + (chunk >> 3) * kHalfBytes + i * 128 + (((chunk & 7) ^ (i & 7)) << 4)) = v;
  }
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// three-input maximum (one instruction on sm_100) and packed two-lane fp32 arithmetic: they halve
// the instruction count of the row maximum, the score scaling and the row sum
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1) {
  asm("{\n\t.reg .b64 ra, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\t"
      "add.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1));
}

// exp2 on the FMA pipe for a share of the scores: floor via a round-down add of 1.5 * 2^23, a cubic
// for 2^frac (relative error 8.6e-5, far below the bf16 rounding of P), exponent added as an integer.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -125.f);
  float r;
  asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(x), "f"(12582912.f));
  const float f = x - (r - 12582912.f);            // fraction in [0, 1)
  float pl = __fmaf_rn(f, 0.07706618f, 0.22764593f);
  pl = __fmaf_rn(pl, f, 0.69511658f);
  pl = __fmaf_rn(pl, f, 1.f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(r) << 23));
}
#ifndef LLNV_ATTN_POLY_MOD
#define LLNV_ATTN_POLY_MOD 8        // every 8th score takes the FMA-pipe exp2 (measured best; 4 is already slower, 0 = none)
#endif

// bf16 window: 10 warps put three warps on some schedulers, whose 16 K-register files then allow 168
// registers per thread.  NVFP4 window: 16 warps start with 128 registers each and re-divide them.
template <bool FUSED>
__global__ void __launch_bounds__(FUSED ? kThreadsFused : kThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const AttnParams p,
                 const __grid_constant__ KvTable tab) {
  pdl_wait();
  constexpr int kSoftmaxWarp0 = FUSED ? 4 : 2;       // first softmax warp (its TMEM lane quarter is warp % 4)
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + kBarOff);
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + kStages;
  uint64_t* v_full = k_empty + kStages;
  uint64_t* v_empty = v_full + kStages;
  uint64_t* s_full = v_empty + kStages;        // [2 halves]
  uint64_t* p_ready = s_full + 2;              // [2 halves]
  uint64_t* pv_done = p_ready + 2;             // [2 halves]
  uint64_t* kc_full = pv_done + 2;             // [kStages] code tiles of a K stage have landed (NVFP4 window)
  uint64_t* vc_full = kc_full + kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(vc_full + kStages);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, head = blockIdx.y;
  const int nt_all = (int)((p.Lk + kBK - 1) / kBK);
  int j0 = (int)((int64_t)blockIdx.z * nt_all / p.nsplit);                  // first key tile of this split
  int nt = (int)((int64_t)(blockIdx.z + 1) * nt_all / p.nsplit) - j0;       // >= 1: the host keeps nsplit <= nt_all
  bool partial = p.part_o != nullptr;
  if (p.tail_cut > 0) {
    if (qt + (int)gridDim.x * head < p.tail_first) {
      if (blockIdx.z != 0) return;             // whole item, done by its z = 0 CTA (nothing is set up yet: the CTA just leaves)
      partial = false;
    } else {
      j0 = blockIdx.z == 0 ? 0 : p.tail_cut;
      nt = blockIdx.z == 0 ? p.tail_cut : nt_all - p.tail_cut;
    }
  }
  const int n_half = ((int64_t)qt * kBQ + kHQ < p.Lq) ? 2 : 1;     // the second half may lie entirely beyond Lq
  // key tiles [0, nd) of this split hold cached keys and are built by the decode warps, the rest come from TMA
  int nd = 0;
  if (FUSED) {
    const int64_t cached_tiles = (p.n_cached + kBK - 1) / kBK - j0;
    nd = cached_tiles <= 0 ? 0 : (cached_tiles < nt ? (int)cached_tiles : nt);
  }

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && p.status && atomicCAS(p.status, 0u, 2u) == 0u) p.status[1] = 901u;
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&kc_full[i], 1);
      mbar_init(&vc_full[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    *abort_flag = 0u;
    fence_barrier_init();
    prefetch_tensormap(&tmQ);
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
    prefetch_tensormap(&tmO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // NVFP4 window: the register file is re-divided at the top of every warpgroup's branch (all four warps of
  // a warpgroup execute the same instruction; an increase waits for the other warpgroups' releases):
  // 16 warps x 32 x 128 registers at launch = 128 x (56 + 104 + 2 x 176).
  if (FUSED && warp < 4) setmaxnreg_dec<56>();

  if (warp == 0 || (FUSED && warp == 2)) {
    // ------------------------------------------------------------------ TMA producer
    // bf16 window: warp 0 loads Q, then K and V tile by tile.  NVFP4 window: warp 0 loads Q and feeds the K
    // stages, warp 2 feeds the V stages, so that neither side queues behind the other's stage becoming free.
    const bool do_k = warp == 0, do_v = FUSED ? warp == 2 : true;
    if (elect_one()) {
      const int col = head * kD;
      if (do_k) {
        mbar_arrive_expect_tx(q_full, n_half * kTileBytes);
        for (int h = 0; h < n_half; ++h) {
          tma_load_2d(smem + kQOff + h * kTileBytes, &tmQ, col, qt * kBQ + h * kHQ, q_full);
          tma_load_2d(smem + kQOff + h * kTileBytes + kHalfBytes, &tmQ, col + 64, qt * kBQ + h * kHQ, q_full);
        }
      }
      // (block, token) of the first key of tile j, advanced tile by tile
      int b0 = FUSED ? (int)(((int64_t)j0 * kBK) / p.block_tokens) : 0;
      int tok0 = FUSED ? (int)((int64_t)j0 * kBK - (int64_t)b0 * p.block_tokens) : 0;
      for (int j = 0; j < nt; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (uint32_t)((j / kStages) & 1);
        if (j < nd) {
          // a tile the decode warps build: its codes go into the tail of the (free) stage, one box of 128 token
          // rows per cache block the tile touches; rows beyond a block's end arrive as zeros and are not used
          const bool two = tok0 + kBK > p.block_tokens && (int64_t)(b0 + 1) * p.block_tokens < p.n_cached;
          const uint32_t bytes = two ? 2 * kCodeBytes : kCodeBytes;
          if (do_k) {
            mbar_wait(&k_empty[s], ph ^ 1u, abort_flag, p.status, 102u);
            mbar_arrive_expect_tx(&kc_full[s], bytes);
            tma_load_2d(smem + kKOff + s * kTileBytes + kCodeOff, &tab.k_codes[b0], head * 64, tok0, &kc_full[s]);
            if (two) tma_load_2d(smem + kKOff + s * kTileBytes + kCodeOff + kCodeBytes, &tab.k_codes[b0 + 1], head * 64, 0, &kc_full[s]);
          }
          if (do_v) {
            mbar_wait(&v_empty[s], ph ^ 1u, abort_flag, p.status, 103u);
            mbar_arrive_expect_tx(&vc_full[s], bytes);
            tma_load_2d(smem + kVOff + s * kTileBytes + kCodeOff, &tab.v_codes[b0], head * 64, tok0, &vc_full[s]);
            if (two) tma_load_2d(smem + kVOff + s * kTileBytes + kCodeOff + kCodeBytes, &tab.v_codes[b0 + 1], head * 64, 0, &vc_full[s]);
          }
          tok0 += kBK;
          if (tok0 >= p.block_tokens) { tok0 -= p.block_tokens; ++b0; }
          continue;
        }
        // row of the tile's first key in the tensor the K / V maps describe (the whole window, or the current chunk)
        const int krow = (j0 + j) * kBK - (FUSED ? (int)p.n_cached : 0);
        if (do_k) {
          mbar_wait(&k_empty[s], ph ^ 1u, abort_flag, p.status, 100u);
          mbar_arrive_expect_tx(&k_full[s], kTileBytes);
          tma_load_2d(smem + kKOff + s * kTileBytes, &tmK, col, krow, &k_full[s]);
          tma_load_2d(smem + kKOff + s * kTileBytes + kHalfBytes, &tmK, col + 64, krow, &k_full[s]);
        }
        if (do_v) {
          mbar_wait(&v_empty[s], ph ^ 1u, abort_flag, p.status, 101u);
          mbar_arrive_expect_tx(&v_full[s], kTileBytes);
          tma_load_2d(smem + kVOff + s * kTileBytes, &tmV, col, krow, &v_full[s]);
          tma_load_2d(smem + kVOff + s * kTileBytes + kHalfBytes, &tmV, col + 64, krow, &v_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(kHQ, kBK, 0, 0);     // A, B K-major
      constexpr uint32_t idesc_pv = make_idesc_bf16(kHQ, kD, 0, 1);      // B (V) MN-major

      auto issue_qk = [&](int t, int h) {
        const int s = t % kStages;
        const uint32_t q_addr = smem_u32(smem + kQOff + h * kTileBytes);
        const uint32_t k_addr = smem_u32(smem + kKOff + s * kTileBytes);
        const uint32_t d_tmem = tmem_base + kSCol + 128 * h;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // 16 channels per MMA: 32 bytes along the swizzled 128-byte row, second half after 4 steps
          const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
          mma_f16_ss(d_tmem, make_kmajor_sw128_desc(q_addr + off), make_kmajor_sw128_desc(k_addr + off), idesc_qk, ks != 0);
        }
        tc_commit(&s_full[h]);
        if (h == n_half - 1) tc_commit(&k_empty[s]);
      };

      mbar_wait(q_full, 0u, abort_flag, p.status, 201u);
      mbar_wait(&k_full[0], 0u, abort_flag, p.status, 200u);
      tc_fence_after();
      for (int h = 0; h < n_half; ++h) issue_qk(0, h);
      for (int j = 0; j < nt; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (uint32_t)((j / kStages) & 1);
        mbar_wait(&v_full[s], ph, abort_flag, p.status, 203u);
        const uint32_t v_addr = smem_u32(smem + kVOff + s * kTileBytes);
        for (int h = 0; h < n_half; ++h) {
          mbar_wait(&p_ready[h], (uint32_t)(j & 1), abort_flag, p.status, 202u);
          tc_fence_after();
          const uint32_t p_tmem = tmem_base + kSCol + 128 * h;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            // 16 keys per MMA: P columns 8*ks..8*ks+7 (two bf16 per column), V rows 16*ks.. (2048 bytes apart)
            // V is MN-major: 64 channels contiguous per key row, the second 64 channels one half-tile further
            const uint64_t v_desc = make_smem_desc(v_addr + ks * 2048, kHalfBytes, 1024, 2);
            mma_f16_ts(tmem_base + kOCol + 128 * h, p_tmem + 8 * ks, v_desc, idesc_pv, (j | ks) != 0);
          }
          tc_commit(&pv_done[h]);
          if (h == n_half - 1) tc_commit(&v_empty[s]);
          if (j + 1 < nt) {
            if (h == 0) {
              mbar_wait(&k_full[(j + 1) % kStages], (uint32_t)(((j + 1) / kStages) & 1), abort_flag, p.status, 204u);
              tc_fence_after();
            }
            issue_qk(j + 1, h);
          }
        }
      }
    }
  } else if (FUSED && warp >= 12) {
    // ------------------------------------------------------------------ NVFP4 decode (warps 12..15)
    // Thread i builds key row i of every tile: first the K stage (the MMAs need it first), then the V stage.
    // (Two groups of 64 threads building K and V side by side, two rows per thread, measured 9 % slower: the
    // K tile is on the critical path and took twice as long.)
    setmaxnreg_dec<104>();
    const int i = (int)threadIdx.x - 384;               // key row of the tile this thread builds; also its table entry
    const int H = p.heads;
    const int T = p.block_tokens;
    const int n_cached = (int)p.n_cached, Lk = (int)p.Lk;      // the host keeps the window below 2^31 keys
    uint8_t* tabs = smem + kTabOff;                       // slot * 4096 + (K: 0, V: 2048) + entry * 16
    // (block, token) of the first key of the tile being fetched, advanced tile by tile (no divisions in the loop)
    int fb = (int)(((int64_t)j0 * kBK) / T);
    int ft = (int)((int64_t)j0 * kBK - (int64_t)fb * T);
    int fkey = j0 * kBK;
    // where key row i of the next tile lives, and its scale bytes (global loads, consumed one tile later)
    auto fetch = [&](RowInfo& r) {
      const int key = fkey + i;
      if (key >= n_cached) {
        r.where = key - n_cached;
        r.kind = key < Lk ? 1 : 2;
      } else {
        const bool second = ft + i >= T;                  // the row lies in the next cache block: second staged code tile
        const int b = second ? fb + 1 : fb;
        const int tok = second ? ft + i - T : ft + i;
        r.kind = 0;
        r.where = (second ? 128 + tok : i) | ((b % kTabSlots) << 8);
        const int row = tok * H + head;                   // row of the block: token-major, head-minor
        const int sf_off = (row >> 7) * 1024 + (row & 31) * 16 + ((row & 127) >> 5) * 4;   // scale columns 0..3; 4..7 are 512 bytes on
        r.ksf[0] = __ldg(reinterpret_cast<const uint32_t*>(tab.k_sf[b] + sf_off));
        r.ksf[1] = __ldg(reinterpret_cast<const uint32_t*>(tab.k_sf[b] + sf_off + 512));
        r.vsf[0] = __ldg(reinterpret_cast<const uint32_t*>(tab.v_sf[b] + sf_off));
        r.vsf[1] = __ldg(reinterpret_cast<const uint32_t*>(tab.v_sf[b] + sf_off + 512));
      }
      fkey += kBK;
      ft += kBK;
      if (ft >= T) { ft -= T; ++fb; }
    };
    // one of K / V of a tile: expand the staged codes (or copy the current chunk's rows) into stage `st`
    auto build = [&](const RowInfo& row, int kv, uint32_t sf0, uint32_t sf1, uint8_t* st, uint64_t* codes_full, uint64_t* full,
                     uint32_t ph) {
      // the stage is free and its code tiles have landed (the producer waited for the stage before it loaded them)
      mbar_wait(codes_full, ph, abort_flag, p.status, 400u + kv);
      uint32_t w[16];
      if (row.kind == 0) {
        // 64-byte rows, 16-byte chunks XOR-swizzled with bits 1-2 of the row index (TMA's 64-byte swizzle)
        const int cr = row.where & 0xFF;
        const uint8_t* src = st + kCodeOff + cr * 64;
        const int sw = (cr >> 1) & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 v4 = *reinterpret_cast<const uint4*>(src + ((c ^ sw) << 4));
          w[4 * c] = v4.x; w[4 * c + 1] = v4.y; w[4 * c + 2] = v4.z; w[4 * c + 3] = v4.w;
        }
      }
      // Both barriers are executed by all 128 threads outside any divergent branch (a tile that mixes cache rows and
      // current-chunk rows splits a warp between the branches above and below; bar.sync needs converged warps).
      __syncwarp();
      asm volatile("bar.sync 1, 128;" ::: "memory");      // every thread holds its codes: the stage's tail may be overwritten
      if (row.kind == 0) {
        decode_row(w, sf0, sf1, tabs + (row.where >> 8) * 4096 + kv * 2048, st, i);
      } else {
        const uint16_t* src = nullptr;
        if (row.kind == 1) src = (kv ? p.v_cur + (int64_t)row.where * p.ldv : p.k_cur + (int64_t)row.where * p.ldk) + (int64_t)head * kD;
        copy_row(src, st, i);
      }
      fence_proxy_async();
      __syncwarp();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (i == 0) mbar_arrive(full);
    };
    // decode tables exist for cache blocks up to `built`; (lb, lt) = (block, token) of the last key of the current tile
    int built = fb - 1;
    int lb = (int)(((int64_t)j0 * kBK + kBK - 1) / T);
    int lt = (int)((int64_t)j0 * kBK + kBK - 1 - (int64_t)lb * T);
    const int last_block = n_cached > 0 ? (n_cached - 1) / T : 0;
    RowInfo nxt;
    nxt.kind = 2;
    if (nd > 0) fetch(nxt);
    for (int j = 0; j < nd; ++j) {
      const int s = j % kStages;
      const uint32_t ph = (uint32_t)((j / kStages) & 1);
      const RowInfo row = nxt;
      if (j + 1 < nd) fetch(nxt);                         // in flight while this tile is decoded
      const int b_hi = lb < last_block ? lb : last_block;
      lt += kBK;
      if (lt >= T) { lt -= T; ++lb; }
      if (b_hi > built) {               // the same for all 128 threads; the first barrier of `build` publishes the tables
        for (int b = built + 1; b <= b_hi; ++b) {
          uint8_t* tb = tabs + (b % kTabSlots) * 4096;
          *reinterpret_cast<uint4*>(tb + i * 16) = decode_table_entry((uint32_t)i, __fmul_rn(__ldg(tab.k_amax[b]), p.inv_denom));
          *reinterpret_cast<uint4*>(tb + 2048 + i * 16) = decode_table_entry((uint32_t)i, __fmul_rn(__ldg(tab.v_amax[b]), p.inv_denom));
        }
        built = b_hi;
      }
#pragma unroll 1
      for (int kv = 0; kv < 2; ++kv)                      // K, then V: one copy of the build code
        build(row, kv, kv ? row.vsf[0] : row.ksf[0], kv ? row.vsf[1] : row.ksf[1], smem + (kv ? kVOff : kKOff) + s * kTileBytes,
              kv ? &vc_full[s] : &kc_full[s], kv ? &v_full[s] : &k_full[s], ph);
    }
  } else if (warp >= kSoftmaxWarp0 && warp < kSoftmaxWarp0 + 8) {
    // ------------------------------------------------------------------ softmax + epilogue
    if (FUSED) setmaxnreg_inc<176>();
    const int q = warp & 3;
    const int half = warp >= kSoftmaxWarp0 + 4 ? 1 : 0;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const float c = p.scale_log2;
    if (half < n_half) {
    float m = -INFINITY;          // running maximum of raw scores used as the exponent offset
    float l = 0.f;                // running sum of exp
    for (int j = 0; j < nt; ++j) {
      const uint32_t s_tmem = tmem_base + lane_base + kSCol + 128 * half;
      mbar_wait(&s_full[half], (uint32_t)(j & 1), abort_flag, p.status, 300u);
      tc_fence_after();
      uint32_t sr[4][32];
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_ld32(s_tmem + 32 * g, sr[g]);
      tmem_ld_wait();
      const int valid = (int)min((int64_t)kBK, p.Lk - (int64_t)(j0 + j) * kBK);
      if (valid < kBK) {                               // only the last key tile can be ragged
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int nv = valid - 32 * g;                // valid columns of this group of 32
          const uint32_t keep = nv >= 32 ? 0xFFFFFFFFu : (nv <= 0 ? 0u : ((1u << nv) - 1u));
#pragma unroll
          for (int i = 0; i < 32; ++i) sr[g][i] = ((keep >> i) & 1u) ? sr[g][i] : 0xFF800000u;      // -inf
        }
      }
      // row maximum with eight independent chains
      float mx[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx[i] = -INFINITY;
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx[(i >> 1) & 7] = fmax3(mx[(i >> 1) & 7], __uint_as_float(sr[g][i]), __uint_as_float(sr[g][i + 1]));
      const float mt = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
      // lazy rescale: keep the old offset unless this tile's maximum exceeds it by more than 2^8
      const bool grow = (mt - m) * c > 8.f;           // also true for the first tile (m = -inf)
      if (__any_sync(0xFFFFFFFFu, grow && j > 0)) {
        // all PV products issued so far must have landed in O before it is rescaled
        mbar_wait(&pv_done[half], (uint32_t)((j - 1) & 1), abort_flag, p.status, 301u);
        tc_fence_after();
        const float m_new = grow ? mt : m;
        const float alpha = ex2((m - m_new) * c);
        l *= alpha;
        m = m_new;
#pragma unroll 1
        for (int g = 0; g < 4; ++g) {
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_base + kOCol + 128 * half + 32 * g, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tmem_base + lane_base + kOCol + 128 * half + 32 * g, o);
        }
        tmem_st_wait();
      } else if (grow) {
        m = mt;                                        // first tile: nothing accumulated yet
      }
      const float mc = m * c;
      const float nmc = -mc;
      float rsum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};      // four packed accumulators (even / odd columns)
      uint32_t pk0[32], pk1[32];
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0, x1;
          fma2(x0, x1, __uint_as_float(sr[g][i]), __uint_as_float(sr[g][i + 1]), c, nmc);
          constexpr int kMod = LLNV_ATTN_POLY_MOD;
          const float p0 = ex2(x0);
          const float p1 = (kMod > 0 && (i + 1) % kMod == kMod - 1) ? ex2_poly(x1) : ex2(x1);
          const int a = ((i >> 1) & 3) * 2;
          add2(rsum[a], rsum[a + 1], p0, p1);
          const uint32_t packed = pack2(p0, p1);
          if (g < 2) pk0[(g * 32 + i) >> 1] = packed; else pk1[((g - 2) * 32 + i) >> 1] = packed;
        }
      const float rs = ((rsum[0] + rsum[1]) + (rsum[2] + rsum[3])) + ((rsum[4] + rsum[5]) + (rsum[6] + rsum[7]));
      l += rs;
      tmem_st32(s_tmem, pk0);
      tmem_st32(s_tmem + 32, pk1);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[half]);
    }
    // ---- epilogue: O / l -> bf16 -> swizzled staging (the Q tile's shared memory) -> TMA store
    mbar_wait(&pv_done[half], (uint32_t)((nt - 1) & 1), abort_flag, p.status, 302u);
    tc_fence_after();
    const int row0 = qt * kBQ + half * kHQ + q * 32;
    if (partial) {
      // one of several key splits: unnormalised fp32 output and (m, l) for the combine kernel
      const int64_t grow = (int64_t)row0 + lane;
      const int64_t slot = ((int64_t)blockIdx.z * p.Lq + grow) * p.heads + head;
      float4* dst = reinterpret_cast<float4*>(p.part_o + slot * kD);
#pragma unroll 1
      for (int g = 0; g < 4; ++g) {
        uint32_t o[32];
        tmem_ld32(tmem_base + lane_base + kOCol + 128 * half + 32 * g, o);
        tmem_ld_wait();
        if (grow < p.Lq) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[g * 8 + i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]), __uint_as_float(o[4 * i + 2]),
                                         __uint_as_float(o[4 * i + 3]));
        }
      }
      if (grow < p.Lq) *reinterpret_cast<float2*>(p.part_ml + slot * 2) = make_float2(m, l);
    } else {
    const float inv_l = 1.f / l;
    uint32_t amax2 = 0u;          // packed running max of |out| (bf16 pairs; the magnitudes compare as integers)
#pragma unroll 1
    for (int dh = 0; dh < 2; ++dh) {
      uint32_t o[2][32];
      tmem_ld32(tmem_base + lane_base + kOCol + 128 * half + 64 * dh, o[0]);
      tmem_ld32(tmem_base + lane_base + kOCol + 128 * half + 64 * dh + 32, o[1]);
      tmem_ld_wait();
      uint8_t* buf = smem + kQOff + half * kTileBytes + dh * kHalfBytes + q * 4096;      // 32 rows x 128 bytes
#pragma unroll
      for (int v8 = 0; v8 < 8; ++v8) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int cc = v8 * 8 + 2 * e;
          const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[cc >> 5][cc & 31]) * inv_l,
                                                          __uint_as_float(o[(cc + 1) >> 5][(cc + 1) & 31]) * inv_l);
          w[e] = *reinterpret_cast<const uint32_t*>(&b2);
          amax2 = __vmaxu2(amax2, w[e] & 0x7FFF7FFFu);
        }
        *reinterpret_cast<uint4*>(buf + lane * 128 + ((v8 ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0 && row0 < p.Lq) {
        tma_store_2d(&tmO, buf, head * kD + dh * 64, row0);
        bulk_commit();
      }
    }
    if (p.out_amax) {
      // rows at or beyond Lq are not written (the TMA store clips them) and must not count
      float a = row0 + lane < p.Lq ? __uint_as_float(max(amax2 & 0xFFFFu, amax2 >> 16) << 16) : 0.f;
      a = warp_max(a);
      if (lane == 0 && a > 0.f) atomic_max_nonneg(p.out_amax, a);
    }
    if (lane == 0) bulk_wait<0>();
    }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Merges the key splits: out = sum_z 2^((m_z - M) c) O_z / sum_z 2^((m_z - M) c) l_z with M = max_z m_z.
// One warp per (query row, head); a lane owns four of the 128 channels.
__global__ void __launch_bounds__(256) attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                int nsplit, int64_t Lq, int heads, float scale_log2,
                                                                uint16_t* __restrict__ out, int64_t ldo, float* __restrict__ out_amax,
                                                                int tail_first, int q_tiles) {
  pdl_wait();
  const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);      // row * heads + head
  const int lane = threadIdx.x & 31;
  if (unit >= Lq * heads) return;
  // tail balancing: only the items that were cut have partial results (the others wrote their output themselves)
  if (tail_first >= 0 && (int)((unit / heads) / kBQ) + q_tiles * (int)(unit % heads) < tail_first) return;
  const int64_t stride = Lq * heads;
  float mmax = -INFINITY;
  for (int z = 0; z < nsplit; ++z) mmax = fmaxf(mmax, __ldg(part_ml + (z * stride + unit) * 2));
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float lsum = 0.f;
  for (int z = 0; z < nsplit; ++z) {
    const float2 ml = __ldg(reinterpret_cast<const float2*>(part_ml + (z * stride + unit) * 2));
    const float w = exp2f((ml.x - mmax) * scale_log2);
    const float4 o = __ldg(reinterpret_cast<const float4*>(part_o + (z * stride + unit) * kD) + lane);
    acc.x = __fmaf_rn(w, o.x, acc.x);
    acc.y = __fmaf_rn(w, o.y, acc.y);
    acc.z = __fmaf_rn(w, o.z, acc.z);
    acc.w = __fmaf_rn(w, o.w, acc.w);
    lsum = __fmaf_rn(w, ml.y, lsum);
  }
  const float inv = 1.f / lsum;
  const int64_t row = unit / heads;
  const int head = (int)(unit % heads);
  uint2 packed;
  packed.x = pack2(acc.x * inv, acc.y * inv);
  packed.y = pack2(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(out + row * ldo + (int64_t)head * kD + lane * 4) = packed;
  if (out_amax) {
    const uint32_t m2 = __vmaxu2(packed.x & 0x7FFF7FFFu, packed.y & 0x7FFF7FFFu);
    const float a = warp_max(__uint_as_float(max(m2 & 0xFFFFu, m2 >> 16) << 16));
    if (lane == 0 && a > 0.f) atomic_max_nonneg(out_amax, a);
  }
}

}  // namespace
}  // namespace llnv

using namespace llnv;

// Tail balancing.  `items` (query tile, head) CTAs of `nt` key tiles each on `sms` SMs run floor(items / sms) full
// waves and then r = items % sms CTAs on an otherwise idle device.  Cutting each of those r items at key tile
// c = r * nt / sms gives r long CTAs (c tiles) and r short ones (nt - c tiles) that the hardware scheduler, which
// hands the next CTA to whichever SM frees up, packs onto the sms - r remaining SMs: the last wave then lasts about c
// tile times instead of nt.  Returns c, or 0 when there is no last partial wave or the saving is below 5 %.
static int tail_cut_for(int64_t items, int64_t nt, int sms) {
  const int64_t r = items % sms;
  if (items <= sms || r == 0 || nt < 16) return 0;
  int64_t c = (r * nt + sms - 1) / sms + 1;            // one extra tile pays for the second set-up of the short CTAs
  if (c < 4) c = 4;
  if (c > nt - 4) return 0;
  const int64_t before = (items / sms + 1) * nt, after = (items / sms) * nt + c;
  return (before - after) * 20 >= before ? (int)c : 0;
}

extern "C" int llnv_attention_key_splits(int64_t Lq, int64_t Lk, int heads) {
  if (Lq <= 0 || Lk <= 0 || heads <= 0) return 1;
  const int64_t ctas = ((Lq + kBQ - 1) / kBQ) * heads;
  const int64_t nt = (Lk + kBK - 1) / kBK;
  const int sms = sm_count();
  if (sms > 0 && ctas > sms && tail_cut_for(ctas, nt, sms) > 0) return LLNV_ATTN_SPLIT_TAIL;
  if (sms <= 0 || 2 * ctas > sms) return 1;                 // the grid already fills most of the device
  int64_t splits = sms / ctas;
  // every split should still run a few key tiles, so that the set-up and the combine pass stay small
  splits = splits < nt / 4 ? splits : nt / 4;
  splits = splits < 16 ? splits : 16;
  return (int)(splits < 1 ? 1 : splits);
}

extern "C" int64_t llnv_attention_workspace_bytes(int64_t Lq, int heads, int key_splits) {
  if (key_splits == LLNV_ATTN_SPLIT_TAIL) key_splits = 2;
  if (key_splits <= 1 || Lq <= 0 || heads <= 0) return 0;
  return (int64_t)key_splits * Lq * heads * (kD + 2) * (int64_t)sizeof(float);
}

namespace {

// Shared host side of the two entry points.  kv == nullptr: k / v are the whole window (bf16).  Otherwise the window
// is kv's cache blocks (n_cached keys) followed by the bf16 tensors k / v of Lk - n_cached keys.
int attention_launch(const void* q, int64_t Lq, int64_t ldq, const void* k, const void* v, int64_t Lk, int64_t ldk, int64_t ldv,
                     int heads, float scale, void* out, int64_t ldo, int key_splits, void* workspace, int64_t workspace_bytes,
                     float* out_amax, const KvTable* kv, int64_t n_cached, int block_tokens, float inv_denom, cudaStream_t stream,
                     const char* who) {
  int tail_cut = 0;
  if (key_splits == LLNV_ATTN_SPLIT_TAIL) {
    const int sms = sm_count();
    if (sms > 0 && Lq > 0 && Lk > 0) tail_cut = tail_cut_for(((Lq + kBQ - 1) / kBQ) * heads, (Lk + kBK - 1) / kBK, sms);
    if (tail_cut > 0)
      LLNV_REQUIRE(workspace != nullptr && ((uintptr_t)workspace & 15) == 0 &&
                       workspace_bytes >= llnv_attention_workspace_bytes(Lq, heads, LLNV_ATTN_SPLIT_TAIL),
                   "%s: tail balancing needs a 16-byte aligned workspace of llnv_attention_workspace_bytes() bytes", who);
    key_splits = 1;
  }
  LLNV_REQUIRE(key_splits >= 1 && key_splits <= 64, "%s: key_splits must be in 1..64 or LLNV_ATTN_SPLIT_TAIL (got %d)", who, key_splits);
  LLNV_REQUIRE(Lk <= 0 || key_splits <= (Lk + kBK - 1) / kBK, "%s: more key splits (%d) than key tiles of 128", who, key_splits);
  if (key_splits > 1) {
    LLNV_REQUIRE(workspace != nullptr && ((uintptr_t)workspace & 15) == 0 &&
                     workspace_bytes >= llnv_attention_workspace_bytes(Lq, heads, key_splits),
                 "%s: key splits need a 16-byte aligned workspace of llnv_attention_workspace_bytes() bytes", who);
  }
  const int64_t L_cur = Lk - n_cached;               // keys held in bf16
  LLNV_REQUIRE(q && out && (L_cur == 0 || (k && v)), "%s: null pointer", who);
  LLNV_REQUIRE(Lq >= 0 && Lk > 0 && L_cur >= 0 && heads > 0, "%s: need Lq >= 0, Lk > 0, heads > 0 (Lq=%lld Lk=%lld heads=%d)", who,
               (long long)Lq, (long long)Lk, heads);
  const int64_t C = (int64_t)heads * kD;
  LLNV_REQUIRE(ldq >= C && ldo >= C && ldq % 8 == 0 && ldo % 8 == 0 && (L_cur == 0 || (ldk >= C && ldv >= C && ldk % 8 == 0 && ldv % 8 == 0)),
               "%s: row strides must be >= heads*128 and multiples of 8", who);
  LLNV_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0 && ((uintptr_t)v & 15) == 0 && ((uintptr_t)out & 15) == 0,
               "%s: pointers must be 16-byte aligned", who);
  LLNV_REQUIRE(heads <= 65535, "%s: too many heads", who);
  if (out_amax && !amax_accumulate(1)) LLNV_CUDA(cudaMemsetAsync(out_amax, 0, sizeof(float), stream));
  if (Lq == 0) return LLNV_OK;
  CUtensorMap tmQ, tmK, tmV, tmO;
  int rc = cached_tensor_map(&tmQ, 1, q, (uint64_t)Lq, (uint64_t)C, (uint64_t)ldq, 128, 64, 3);
  if (rc != LLNV_OK) return rc;
  if (L_cur > 0) {
    rc = cached_tensor_map(&tmK, 1, k, (uint64_t)L_cur, (uint64_t)C, (uint64_t)ldk, 128, 64, 3);
    if (rc != LLNV_OK) return rc;
    rc = cached_tensor_map(&tmV, 1, v, (uint64_t)L_cur, (uint64_t)C, (uint64_t)ldv, 128, 64, 3);
    if (rc != LLNV_OK) return rc;
  } else {
    tmK = tmQ;                  // never used: every key tile is built by the decode warps
    tmV = tmQ;
  }
  rc = cached_tensor_map(&tmO, 1, out, (uint64_t)Lq, (uint64_t)C, (uint64_t)ldo, 32, 64, 3);
  if (rc != LLNV_OK) return rc;
  static bool attr_set[2][64] = {};
  int dev = 0;
  LLNV_CUDA(cudaGetDevice(&dev));
  const int fused = kv != nullptr ? 1 : 0;
  if (dev >= 0 && dev < 64 && !attr_set[fused][dev]) {
    if (fused) LLNV_CUDA(cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytesFused));
    else LLNV_CUDA(cudaFuncSetAttribute(attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    attr_set[fused][dev] = true;
  }
  AttnParams p;
  p.Lq = Lq;
  p.Lk = Lk;
  p.heads = heads;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = device_status_word();
  const int zdim = tail_cut > 0 ? 2 : key_splits;     // partial-result slices in the workspace
  p.nsplit = key_splits;
  p.tail_cut = tail_cut;
  p.tail_first = tail_cut > 0 ? (int)((((Lq + kBQ - 1) / kBQ) * heads / sm_count()) * sm_count()) : 0;
  p.part_o = zdim > 1 ? (float*)workspace : nullptr;
  p.part_ml = zdim > 1 ? (float*)workspace + (int64_t)zdim * Lq * heads * kD : nullptr;
  p.out_amax = key_splits > 1 ? nullptr : out_amax;   // with tail balancing the whole items report their own maximum
  p.n_cached = n_cached;
  p.block_tokens = block_tokens > 0 ? block_tokens : 1;
  p.inv_denom = inv_denom;
  p.k_cur = (const uint16_t*)k;
  p.v_cur = (const uint16_t*)v;
  p.ldk = ldk;
  p.ldv = ldv;
  dim3 grid((unsigned)((Lq + kBQ - 1) / kBQ), (unsigned)heads, (unsigned)zdim);
  static const KvTable no_blocks = {};      // the bf16 kernel never reads it
  if (fused) launch_k(attention_kernel<true>, grid, kThreadsFused, kSmemBytesFused, stream, tmQ, tmK, tmV, tmO, p, *kv);
  else launch_k(attention_kernel<false>, grid, kThreads, kSmemBytes, stream, tmQ, tmK, tmV, tmO, p, no_blocks);
  int st = launch_status("attention_kernel");
  if (st != LLNV_OK || zdim == 1) return st;
  const int64_t units = Lq * heads;
  launch_k(attention_combine_kernel, (unsigned)((units + 7) / 8), 256, 0, stream, p.part_o, p.part_ml, zdim, Lq, heads, p.scale_log2,
           (uint16_t*)out, ldo, out_amax, tail_cut > 0 ? p.tail_first : -1, (int)grid.x);
  return launch_status("attention_combine_kernel");
}

}  // namespace

extern "C" int llnv_attention_bf16_ex(const void* q, int64_t Lq, int64_t ldq, const void* k, const void* v, int64_t Lk,
                                      int64_t ldk, int64_t ldv, int heads, float scale, void* out, int64_t ldo,
                                      int key_splits, void* workspace, int64_t workspace_bytes, float* out_amax,
                                      llnv_stream_t stream) {
  LLNV_REQUIRE(k && v, "llnv_attention_bf16: null pointer");
  return attention_launch(q, Lq, ldq, k, v, Lk, ldk, ldv, heads, scale, out, ldo, key_splits, workspace, workspace_bytes, out_amax,
                          nullptr, 0, 0, 0.f, (cudaStream_t)stream, "llnv_attention_bf16");
}

extern "C" int llnv_attention_nvfp4kv(const void* q, int64_t Lq, int64_t ldq, const void* const* k_codes, const void* const* k_sf,
                                      const float* const* k_amax, const void* const* v_codes, const void* const* v_sf,
                                      const float* const* v_amax, int num_blocks, int block_token_size, float e2m1_max,
                                      float e4m3_max, const void* k_cur, const void* v_cur, int64_t L_cur, int64_t ldk, int64_t ldv,
                                      int heads, float scale, void* out, int64_t ldo, int key_splits, void* workspace,
                                      int64_t workspace_bytes, float* out_amax, llnv_stream_t stream) {
  const char* who = "llnv_attention_nvfp4kv";
  LLNV_REQUIRE(num_blocks >= 0 && num_blocks <= kMaxKvBlocks, "%s: 0 to %d cache blocks (got %d)", who, kMaxKvBlocks, num_blocks);
  LLNV_REQUIRE(L_cur >= 0 && (num_blocks > 0 || L_cur > 0), "%s: the window is empty", who);
  if (num_blocks == 0)
    return attention_launch(q, Lq, ldq, k_cur, v_cur, L_cur, ldk, ldv, heads, scale, out, ldo, key_splits, workspace, workspace_bytes,
                            out_amax, nullptr, 0, 0, 0.f, (cudaStream_t)stream, who);
  LLNV_REQUIRE(k_codes && k_sf && k_amax && v_codes && v_sf && v_amax, "%s: null pointer table", who);
  LLNV_REQUIRE(block_token_size >= 128 && heads > 0, "%s: block_token_size must be at least 128 (got %d) and heads positive", who,
               block_token_size);
  LLNV_REQUIRE(e2m1_max > 0 && e4m3_max > 0, "%s: e2m1_max and e4m3_max must be positive", who);
  static thread_local KvTable tab;          // 4.5 KiB, copied into the launch parameters
  for (int b = 0; b < num_blocks; ++b) {
    LLNV_REQUIRE(k_codes[b] && k_sf[b] && k_amax[b] && v_codes[b] && v_sf[b] && v_amax[b], "%s: null pointer in block %d", who, b);
    LLNV_REQUIRE(((uintptr_t)k_codes[b] & 15) == 0 && ((uintptr_t)v_codes[b] & 15) == 0 && ((uintptr_t)k_sf[b] & 3) == 0 &&
                     ((uintptr_t)v_sf[b] & 3) == 0,
                 "%s: codes of block %d must be 16-byte, scales 4-byte aligned", who, b);
    tab.k_sf[b] = (const uint8_t*)k_sf[b];
    tab.k_amax[b] = k_amax[b];
    tab.v_sf[b] = (const uint8_t*)v_sf[b];
    tab.v_amax[b] = v_amax[b];
    // byte tensor [tokens, heads * 64], box 128 tokens x 64 bytes, 64-byte swizzle
    int rc = cached_tensor_map(&tab.k_codes[b], 0, k_codes[b], (uint64_t)block_token_size, (uint64_t)heads * 64, (uint64_t)heads * 64, 128, 64, 2);
    if (rc == LLNV_OK) rc = cached_tensor_map(&tab.v_codes[b], 0, v_codes[b], (uint64_t)block_token_size, (uint64_t)heads * 64, (uint64_t)heads * 64, 128, 64, 2);
    if (rc != LLNV_OK) return rc;
  }
  const int64_t n_cached = (int64_t)num_blocks * block_token_size;
  const float inv_denom = (float)(1.0 / ((double)e2m1_max * (double)e4m3_max));
  return attention_launch(q, Lq, ldq, k_cur, v_cur, n_cached + L_cur, ldk, ldv, heads, scale, out, ldo, key_splits, workspace,
                          workspace_bytes, out_amax, &tab, n_cached, block_token_size, inv_denom, (cudaStream_t)stream, who);
}

extern "C" int llnv_attention_bf16(const void* q, int64_t Lq, int64_t ldq, const void* k, const void* v, int64_t Lk,
                                   int64_t ldk, int64_t ldv, int heads, float scale, void* out, int64_t ldo,
                                   llnv_stream_t stream) {
  return llnv_attention_bf16_ex(q, Lq, ldq, k, v, Lk, ldk, ldv, heads, scale, out, ldo, 1, nullptr, 0, nullptr, stream);
}
