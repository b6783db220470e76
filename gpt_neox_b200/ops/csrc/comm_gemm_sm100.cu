// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a, tcgen05 + TMA).
//
// One kernel, same pipeline as gemm_sm100.cu (TMA ring -> tcgen05.mma -> TMEM -> epilogue warps), with two
// extensions that replace the NCCL calls around a column- / row-parallel linear layer:
//
//   * BROADCAST (all-gather -> GEMM).  A few CTAs of the grid do no math: they copy this rank's shard of a
//     row-sharded tensor into slot [rank] of EVERY rank's full-size symmetric buffer with posted peer stores (NVLink
//     writes need no round trip; copy warps inside the GEMM CTAs were measured 10x slower because their loads queue
//     behind the TMA operand traffic), 32 KB pieces at a time in the order the receivers will need them, and bump a
//     per-128-row-block counter in the receiver's memory after each piece.  When an operand of the GEMM is the
//     gathered buffer, a watcher warp in every GEMM CTA turns the counters into a "blocks complete so far" watermark
//     in shared memory and the TMA producer waits -- bounded -- on that before its first load from a block; tiles
//     (or k-steps) are visited local-shard-first, so the arrival of block i+1 overlaps the tensor-core work on
//     block i and every byte crosses NVLink exactly once.  The broadcast may also ride on a GEMM
//     that does not read the tensor (a prefetch: the weight-gradient GEMM of a column-parallel layer then finds the
//     gathered activations complete).
//
//   * PUSH (GEMM -> reduce-scatter).  Row block m of the partial product belongs to rank m / rows_per_rank; the
//     epilogue warps stage each finished 32x64 sub-tile in shared memory and TMA-store it straight into the OWNER's
//     receive buffer, slot [source rank] (128-byte rows, no multicast), so the transfer of tile i overlaps the math
//     of tile i+1; remote owners are served first.  A small second kernel on the owner waits for every source's
//     "all tiles pushed" flag and adds the slots in rank order in fp32 (deterministic), fusing bias and residual.
//
// Flags are 32-bit epochs in the receiver's signal pad, written with st.release.sys after a system fence and read
// with ld.acquire.sys in a loop that gives up after ~2 s, records a status code and lets the kernel drain.
// No multicast of any kind is used.
#include "gemm_common.cuh"
#include "neox_b200.h"
#include <stdlib.h>
#include <string.h>

using namespace gemm;

namespace {

constexpr int MAX_RANKS = 8;
constexpr int COMM_THREADS = 256;                  // GEMM CTA: warp 0 TMA, 1 MMA, 2-5 epilogue, 6 watcher
constexpr int COPY_WARPS = COMM_THREADS / 32;       // copy CTA: every warp copies
constexpr int PIECE_BYTES = 32768;
constexpr int STG_BYTES = 32 * 128;                // one 32-row x 64-column bf16 sub-tile
constexpr int COMM_SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 8 * STG_BYTES + 256 + 1024;
// CTA-pair form (cta_group::2, see gemm_2cta_sm100.cu): each CTA stages 128 rows of A and half of the B tile
constexpr int PSTAGES = 6;
constexpr int PB_STAGE_BYTES = (BN / 2) * BK * 2;
constexpr int PAIR_SMEM_BYTES = PSTAGES * (A_STAGE_BYTES + PB_STAGE_BYTES) + 8 * STG_BYTES + 256 + 1024;

struct OutMaps {
    CUtensorMap m[MAX_RANKS];
};

struct CommParams {
    GemmParams g;
    int world, rank;
    // ---- broadcast job: this rank's shard -> slot [rank] of every rank's gathered buffer
    int bcast;
    int n_copy;                       // CTAs at the end of the grid that only copy
    const uint4* bc_src;              // local shard [rows_per_shard][row_bytes]
    uint4* bc_dst[MAX_RANKS];         // every rank's gathered buffer (peer-mapped)
    unsigned* bc_cnt[MAX_RANKS];      // every rank's per-block arrival flags (peer-mapped)
    unsigned* bc_local_cnt;           // local scratch [world * blocks_per_rank]: pieces sent per block (zero at rest)
    const uint32_t* bc_free_flags;    // local pad: bc_free_flags[dst] >= bc_free_epoch  <=>  dst released its buffer
    uint32_t bc_free_epoch;
    long long shard_bytes;            // bytes of one shard
    long long block_bytes;            // bytes of 128 rows
    int blocks_per_rank;              // 128-row blocks per shard
    int pieces_per_block;
    // ---- dependency of an operand on a gathered buffer
    int a_dep, b_dep;                 // operand A / B is the local gathered buffer: wait for a block before loading
    const unsigned* dep_cnt;          // local arrival flags [world * blocks_per_rank]
    int rows_per_shard;               // rows of the gathered tensor per rank (multiple of 128)
    // ---- push job
    int scatter;                      // 1: epilogue pushes row blocks to their owner's receive buffer
    int rows_per_rank;                // output rows owned by each rank
    const uint32_t* free_flags;       // local pad: free_flags[owner] >= free_epoch  <=>  owner's buffer is reusable
    uint32_t free_epoch;
    // ---- end-of-grid signal
    uint32_t* peer_pad[MAX_RANKS];    // every rank's signal pad (peer-mapped)
    int sig_offset;                   // >= 0: peer_pad[dst][sig_offset + rank] = sig_value when the grid is done
    uint32_t sig_value;
    int sig2_offset;                  // second, independent signal (unused slot for callers that need two)
    uint32_t sig2_value;
    unsigned* counter;                // local CTA-completion counter for the end-of-grid signal
};

struct PeerPads {
    uint32_t* p[MAX_RANKS];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for flag >= epoch (epochs only grow; wrap-around is handled by the signed difference).
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t epoch) {
    if ((int32_t)(ld_acquire_sys(p) - epoch) >= 0) return true;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(p) - epoch) < 0) {
        if (clock64() - t0 > SPIN_LIMIT_CYCLES) return false;
        __nanosleep(64);
    }
    return true;
}
// Called by one thread per CTA after the CTA's last global / peer store (and a __syncthreads()).  The CTA that
// arrives last publishes the value(s) in slot [offset + rank] of every rank's signal pad.
__device__ __forceinline__ void grid_done_signal(unsigned* counter, uint32_t* const* pads, int world, int rank,
                                                 int offset, uint32_t value, int offset2 = -1, uint32_t value2 = 0) {
    __threadfence_system();
    const unsigned old = atomicAdd(counter, 1u);
    if (old == gridDim.x - 1) {
        atomicExch(counter, 0u);
        __threadfence_system();
        for (int dst = 0; dst < world; ++dst) {
            if (offset >= 0) st_release_sys(pads[dst] + offset + rank, value);
            if (offset2 >= 0) st_release_sys(pads[dst] + offset2 + rank, value2);
        }
    }
}

// Scatter epilogue for 32 columns of one row: partial = acc (+ bias) (+ local bf16 addend) as 4 x 16 bytes of bf16.
// Columns beyond N are produced as zeros-or-garbage and clipped by the TMA store.
__device__ __forceinline__ void pack_partial(const uint32_t (&r)[32], int row, int col0, const GemmParams& p,
                                             uint4* out) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    const bool inb = (row < p.M) && (col0 + 32 <= p.N);
    if (inb) {
        if (p.bias) {
            const uint4* b4 = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 b = __ldg(b4 + j);
                const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    v[j * 8 + t * 2] += bf16_lo(w[t]);
                    v[j * 8 + t * 2 + 1] += bf16_hi(w[t]);
                }
            }
        }
        if (p.add) {
            const uint4* a4 = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.add) +
                                                             (long long)row * p.ldadd + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 a = a4[j];
                const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    v[j * 8 + t * 2] += bf16_lo(w[t]);
                    v[j * 8 + t * 2 + 1] += bf16_hi(w[t]);
                }
            }
        }
    } else if (row < p.M) {
        for (int i = 0; i < 32 && col0 + i < p.N; ++i) {
            if (p.bias) v[i] += __bfloat162float(p.bias[col0 + i]);
            if (p.add) v[i] += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.add)[(long long)row * p.ldadd + col0 + i]);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint4 q;
        q.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
        q.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
        q.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
        q.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
        out[j] = q;
    }
}

// PAIR: launched as (2,1,1) clusters; the two CTAs of a cluster compute one 256 x 256 tile with cta_group::2 MMAs
// issued by the even CTA (barrier protocol of gemm_2cta_sm100.cu).  Everything a CTA does on its own -- waiting for
// gathered blocks before loading them, the epilogue of its 128 output rows including the push to the rows' owner,
// the watcher warp, copy CTAs (which come in pairs too) -- is the same in both forms.
template <bool PAIR>
__global__ void __launch_bounds__(COMM_THREADS, 1)
comm_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ OutMaps outm, const CommParams cp) {
    constexpr int NSTG = PAIR ? PSTAGES : STAGES;
    constexpr int BSTG = PAIR ? PB_STAGE_BYTES : B_STAGE_BYTES;
    constexpr int TM = PAIR ? 2 * BM : BM;                       // output rows per tile
    const GemmParams& p = cp.g;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + NSTG * A_STAGE_BYTES;
    uint8_t* sStg = smem + NSTG * (A_STAGE_BYTES + BSTG);
    uint64_t* full = reinterpret_cast<uint64_t*>(sStg + 8 * STG_BYTES);
    uint64_t* empty = full + NSTG;
    uint64_t* tfull = empty + NSTG;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* watermark = reinterpret_cast<volatile int*>(tmem_slot + 1);   // gathered blocks complete so far

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_gemm = gridDim.x - cp.n_copy;            // GEMM CTAs come first, copy CTAs last
    const bool copy_cta = (int)blockIdx.x >= n_gemm;
    const int crank = PAIR ? (int)cluster_ctarank() : 0; // 0 = the CTA that issues the MMAs
    const int unit = PAIR ? (int)blockIdx.x >> 1 : (int)blockIdx.x;      // tile-processing unit: a CTA or a pair
    const int n_units = PAIR ? n_gemm >> 1 : n_gemm;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTG; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], PAIR ? 8 : 4);
        }
        *watermark = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (PAIR) cluster_sync_all();                        // both CTAs' barriers exist before anyone signals across
    if (warp == 1 && !copy_cta) {
        if (PAIR) {
            tmem_alloc_pair(tmem_slot, 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 512);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = copy_cta ? 0u : *tmem_slot;

    const int num_m = (p.M + TM - 1) / TM;
    const int num_n = (p.N + BN - 1) / BN;
    const int ntiles = num_m * num_n;
    const int nk = (p.K + BK - 1) / BK;
    // Rotations: start on the local shard when an operand is being gathered, on the next rank's rows when pushing.
    int m_rot = 0, k_rot = 0;
    if (cp.a_dep && !p.a_mn) m_rot = (cp.rank * cp.rows_per_shard) / TM;
    if ((cp.a_dep && p.a_mn) || (cp.b_dep && p.b_mn)) k_rot = (cp.rank * cp.rows_per_shard) / BK;
    if (cp.scatter) m_rot = (((cp.rank + 1) % cp.world) * cp.rows_per_rank) / TM;

    auto coords = [&](int tile, int& m_blk, int& n_blk) {
        // groups of 2048 rows of tiles walk across N together (the A panel stays in L2)
        constexpr int GM = PAIR ? GROUP_M / 2 : GROUP_M;
        const int per_group = GM * num_n;
        const int group = tile / per_group;
        const int first_m = group * GM;
        const int gsize = min(num_m - first_m, GM);
        const int in_group = tile - group * per_group;
        m_blk = (first_m + in_group % gsize + m_rot) % num_m;
        n_blk = in_group / gsize;
    };

    const int dep_total = cp.world * cp.blocks_per_rank;          // gathered blocks, consumed starting at the local shard
    const int dep_rot = cp.rank * cp.blocks_per_rank;

    if (copy_cta) {
        // ------------------------------------------------------------ copy CTA: broadcast the local shard
        // Phase i sends to rank - i: every rank then receives, in phase i, the shard of rank + i, which is the order
        // in which its own GEMM consumes them, and each phase is a permutation (balanced through the switch).
        const int gw = ((int)blockIdx.x - n_gemm) * COPY_WARPS + warp;
        const int GW = cp.n_copy * COPY_WARPS;
        const int per_dst = cp.blocks_per_rank * cp.pieces_per_block;
        const long long units = (long long)cp.world * per_dst;
        uint32_t freed = 1u << cp.rank;
        for (long long u = gw; u < units; u += GW) {
            const int i = (int)(u / per_dst);
            const int dst = (cp.rank - i + cp.world) % cp.world;
            const int rem = (int)(u - (long long)i * per_dst);
            const int rb = rem / cp.pieces_per_block;
            const int piece = rem - rb * cp.pieces_per_block;
            if (!(freed & (1u << dst))) {
                int okf = 1;
                if (lane == 0) okf = wait_flag(cp.bc_free_flags + dst, cp.bc_free_epoch) ? 1 : 0;
                okf = __shfl_sync(0xffffffffu, okf, 0);
                if (!okf) {
                    if (lane == 0) atomicExch(p.status, 460 + dst);
                    break;
                }
                freed |= 1u << dst;
                __syncwarp();
            }
            const long long off = (long long)rb * cp.block_bytes + (long long)piece * PIECE_BYTES;
            long long len = cp.block_bytes - (long long)piece * PIECE_BYTES;
            if (len > PIECE_BYTES) len = PIECE_BYTES;
            const int nvec = (int)(len >> 4);
            const uint4* __restrict__ s4 = cp.bc_src + (off >> 4);
            uint4* __restrict__ d4 = cp.bc_dst[dst] + (((long long)cp.rank * cp.shard_bytes + off) >> 4);
            int v = lane;
            for (; v + 15 * 32 < nvec; v += 32 * 16) {    // 16 independent 16-byte loads in flight per lane
                uint4 t[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) t[j] = __ldg(s4 + v + j * 32);
#pragma unroll
                for (int j = 0; j < 16; ++j) d4[v + j * 32] = t[j];
            }
            for (; v < nvec; v += 32) d4[v] = __ldg(s4 + v);
            __syncwarp();
            // System-scope releases are serialised GPU-wide (measured: ~0.5 us each, 3000 of them dominated the
            // kernel), so pieces are counted locally at GPU scope and only the warp that completes a 128-row block
            // publishes it to the receiver: one system-scope release per block and destination.
            if (lane == 0) {
                __threadfence();
                unsigned* lc = cp.bc_local_cnt + dst * cp.blocks_per_rank + rb;
                if (atomicAdd(lc, 1u) == (unsigned)cp.pieces_per_block - 1u) {
                    atomicExch(lc, 0u);                     // ready for the next launch
                    __threadfence();
                    red_release_sys_add(cp.bc_cnt[dst] + cp.rank * cp.blocks_per_rank + rb, 1u);
                }
            }
        }
    } else if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int known = 0;                        // watermark value last read
            // Wait until the gathered block holding `row` has arrived (the watcher warp maintains the watermark).
            auto block_ready = [&](int row) -> bool {
                int o = (row >> 7) - dep_rot;
                if (o < 0) o += dep_total;
                if (o < known) return true;
                const long long t0 = clock64();
                for (;;) {
                    known = *watermark;
                    if (known < 0) return false;           // the watcher gave up and reported
                    if (o < known) break;
                    if (clock64() - t0 > SPIN_LIMIT_CYCLES) {
                        atomicExch(p.status, 400 + row / cp.rows_per_shard);
                        return false;
                    }
                    __nanosleep(100);
                }
                __threadfence();
                // the block was written through the generic proxy; TMA reads it through the async proxy
                asm volatile("fence.proxy.async.global;" ::: "memory");
                return true;
            };
            // one load, counted on this CTA's barrier or (PAIR) on the leader's
            auto load = [&](void* dst, const CUtensorMap* m, uint64_t* bar, int x0, int y0) {
                if (PAIR) tma_load_2d_pair(dst, m, bar, x0, y0);
                else tma_load_2d(dst, m, bar, x0, y0);
            };
            constexpr int BN_CTA = PAIR ? BN / 2 : BN;    // B columns this CTA stages
            // Everything the loop needs sits in registers: one thread runs this loop, and at one k-block per ~500
            // clocks a chain of dependent parameter loads, a modulo and branches per iteration is enough to make
            // it the limiter of the whole kernel (measured: tensor pipe 78 % busy against 96 % in the plain kernel).
            const bool a_mn = p.a_mn != 0, b_mn = p.b_mn != 0, a_dep = cp.a_dep != 0, b_dep = cp.b_dep != 0;
            const int dep_rows = cp.rows_per_shard * cp.world;
            const uint32_t tx_bytes = PAIR ? 2 * (A_STAGE_BYTES + PB_STAGE_BYTES) : A_STAGE_BYTES + B_STAGE_BYTES;
            const bool arm = !PAIR || crank == 0;
            for (int tile = unit; tile < ntiles && ok; tile += n_units) {
                int m_blk, n_blk;
                coords(tile, m_blk, n_blk);
                const int m0 = m_blk * TM + crank * BM;   // this CTA's rows of A
                const int n0 = n_blk * BN + crank * BN_CTA;
                int kb = k_rot;
                for (int kk = 0; kk < nk; ++kk) {
                    if (!mbar_wait(&empty[stage], phase ^ 1)) {
                        atomicExch(p.status, 101);
                        ok = false;
                        break;
                    }
                    const int k0 = kb * BK;
                    // y coordinate = row of the operand's 2-D view
                    const int ay = a_mn ? k0 : m0;
                    const int by = b_mn ? k0 : n0;
                    if (a_dep && !block_ready(ay)) { ok = false; break; }
                    if (b_dep) {
                        // an N-side K-major tile of 256 rows spans two 128-row blocks
                        if (!block_ready(by)) { ok = false; break; }
                        if (!PAIR && !b_mn && by + 128 < dep_rows && !block_ready(by + 128)) {
                            ok = false;
                            break;
                        }
                    }
                    if (arm) mbar_expect_tx(&full[stage], tx_bytes);
                    uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
                    uint8_t* b_dst = sB + stage * BSTG;
                    if (!a_mn) {
                        load(a_dst, &tmA, &full[stage], k0, ay);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            load(a_dst + j * (64 * BK * 2), &tmA, &full[stage], m0 + j * 64, ay);
                    }
                    if (!b_mn) {
                        load(b_dst, &tmB, &full[stage], k0, by);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN_CTA / 64; ++j)
                            load(b_dst + j * (64 * BK * 2), &tmB, &full[stage], n0 + j * 64, by);
                    }
                    if (++stage == NSTG) {
                        stage = 0;
                        phase ^= 1;
                    }
                    if (++kb == nk) kb = 0;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && crank == 0) {
            const uint32_t idesc = make_idesc_bf16(TM, BN, p.a_mn, p.b_mn);
            // operand descriptors as in gemm_sm100.cu: constant upper half, one add per operand per MMA
            const uint32_t desc_hi = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), p.a_mn ? 64 * BK * 2 : 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), p.b_mn ? 64 * BK * 2 : 16);
            const uint32_t a_step = (p.a_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            const uint32_t b_step = (p.b_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t bphase = 0;
            bool ok = true;
            for (int tile = unit; tile < ntiles && ok; tile += n_units) {
                if (!mbar_wait(&tempty[buf], bphase ^ 1)) {
                    atomicExch(p.status, 102);
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < nk; ++kb) {
                    if (!mbar_wait(&full[stage], phase)) {
                        atomicExch(p.status, 103);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + stage * (A_STAGE_BYTES >> 4);
                    const uint32_t b_lo = b_lo0 + stage * (BSTG >> 4);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_ss_lohi<PAIR, false>(tmem_d, a_lo + k * a_step, desc_hi, b_lo + k * b_step, desc_hi, idesc,
                                                  (kb | k) != 0);
                    if (PAIR) umma_commit_pair(&empty[stage], 3);
                    else umma_commit(&empty[stage]);
                    if (++stage == NSTG) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                if (PAIR) umma_commit_pair(&tfull[buf], 3);
                else umma_commit(&tfull[buf]);
                buf ^= 1;
                if (buf == 0) bphase ^= 1;
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue warps (2..5)
        const int q = warp & 3;  // tensor-memory lane quarter this warp may read
        int buf = 0;
        uint32_t bphase = 0;
        uint32_t freed = 1u << cp.rank;   // bit o: owner o's receive buffer is known to be reusable
        uint8_t* stg = sStg + q * 2 * STG_BYTES;
        int sbuf = 0;
        // PAIR: both CTAs' epilogue warps free an accumulator buffer on the LEADER's barrier
        const uint32_t tempty_leader0 = PAIR ? cluster_map(smem_u32(&tempty[0]), 0) : 0u;
        for (int tile = unit; tile < ntiles; tile += n_units) {
            int m_blk, n_blk;
            coords(tile, m_blk, n_blk);
            const int mrow0 = m_blk * TM + crank * BM;            // first output row of this CTA
            if (!mbar_wait_warp(&tfull[buf], bphase)) {
                if (lane == 0) atomicExch(p.status, 104);
                break;
            }
            tc_fence_after();
            const int row = mrow0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
            if (!cp.scatter) {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int col0 = n_blk * BN + c * 32;
                    if (col0 >= p.N) break;  // warp-uniform
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + c * 32, r);
                    tmem_wait_ld();
                    if (row < p.M) epilogue_chunk(r, row, col0, p);
                }
            } else {
                const int owner = min(mrow0 / cp.rows_per_rank, cp.world - 1);   // warp-uniform
                if (!(freed & (1u << owner))) {
                    int okf = 1;
                    if (lane == 0) okf = wait_flag(cp.free_flags + owner, cp.free_epoch) ? 1 : 0;
                    okf = __shfl_sync(0xffffffffu, okf, 0);
                    if (!okf) {
                        if (lane == 0) atomicExch(p.status, 440 + owner);
                        break;
                    }
                    freed |= 1u << owner;
                }
                const int lrow0 = mrow0 + q * 32 - owner * cp.rows_per_rank;   // first row of this warp in the slot
#pragma unroll 1
                for (int c = 0; c < BN / 64; ++c) {
                    const int col0 = n_blk * BN + c * 64;
                    if (col0 >= p.N) break;  // warp-uniform
                    uint32_t r0[32], r1[32];
                    tmem_ld_32x32(taddr + c * 64, r0);
                    tmem_ld_32x32(taddr + c * 64 + 32, r1);
                    tmem_wait_ld();
                    uint4 pk[8];
                    pack_partial(r0, row, col0, p, pk);
                    pack_partial(r1, row, col0 + 32, p, pk + 4);
                    // the store issued two chunks ago has finished reading this staging buffer
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                    uint8_t* sb = stg + sbuf * STG_BYTES + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(sb + ((j ^ (lane & 7)) << 4)) = pk[j];
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&outm.m[owner], stg + sbuf * STG_BYTES, col0, lrow0);
                        tma_store_commit();
                    }
                    sbuf ^= 1;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(tempty_leader0 + buf * 8);
                else mbar_arrive(&tempty[buf]);
            }
            buf ^= 1;
            if (buf == 0) bphase ^= 1;
        }
        if (cp.scatter && lane == 0) {
            tma_store_wait<0>();                                   // all pushed tiles are written
            asm volatile("fence.proxy.async.global;" ::: "memory");
        }
    } else if (warp == 6 && (cp.a_dep || cp.b_dep)) {
        // ------------------------------------------------------------ watcher: counters -> watermark
        int W = 0;
        long long t0 = clock64();
        while (W < dep_total) {
            const int o = W + lane;
            bool c = false;
            if (o < dep_total) {
                int blk = o + dep_rot;
                if (blk >= dep_total) blk -= dep_total;
                c = ld_acquire_sys(cp.dep_cnt + blk) != 0u;
            }
            const unsigned m = __ballot_sync(0xffffffffu, c);
            const int n = (m == 0xffffffffu) ? 32 : (__ffs(~m) - 1);      // leading complete blocks
            if (n > 0) {
                W = min(W + n, dep_total);
                if (lane == 0) {
                    __threadfence();
                    *watermark = W;
                }
                t0 = clock64();
            } else {
                if (clock64() - t0 > SPIN_LIMIT_CYCLES) {
                    if (lane == 0) {
                        int blk = W + dep_rot;
                        if (blk >= dep_total) blk -= dep_total;
                        atomicExch(p.status, 400 + blk / cp.blocks_per_rank);
                        *watermark = -1;
                    }
                    break;
                }
                __nanosleep(200);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    // PAIR: no CTA leaves, or frees tensor memory, while its partner may still signal it or run MMAs into it
    if (PAIR) cluster_sync_all();
    if (warp == 1 && !copy_cta) {
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem_base, 512);
        else tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && (cp.sig_offset >= 0 || cp.sig2_offset >= 0))
        grid_done_signal(cp.counter, cp.peer_pad, cp.world, cp.rank, cp.sig_offset, cp.sig_value, cp.sig2_offset,
                         cp.sig2_value);
}

// Copy this rank's shard into its symmetric staging buffer (and, optionally, into its slot of the local gathered
// tensor) and tell every rank it is there.
//   wait  : the buffer was last read by the peers' GEMMs of epoch `need`; done_flags[peer] >= need says they finished
//   copy  : 16-byte vectors, grid-stride
//   signal: last CTA writes `epoch` into slot [sig_offset + rank] of every pad
__global__ void __launch_bounds__(256) publish_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                      uint4* __restrict__ dst2, size_t nvec,
                                                      const uint32_t* done_flags, uint32_t need, PeerPads pads, int world,
                                                      int rank, int sig_offset, uint32_t epoch, unsigned* counter,
                                                      int* status) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        int ok = 1;
        for (int r = 0; r < world && ok; ++r)
            if (r != rank && !wait_flag(done_flags + r, need)) {
                atomicExch(status, 460 + r);
                ok = 0;
            }
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;     // nothing published: the readers' own bounded waits will report it
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = src[i];
        dst[i] = v;
        if (dst2) dst2[i] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) grid_done_signal(counter, pads.p, world, rank, sig_offset, epoch);
}

// Owner side of the reduce-scatter: out[row, col] = sum_src recv[src][row][col] (+ bias[col]) (+ residual[row, col]),
// sources added in rank order in fp32.  Waits for every source's "pushed" flag first; when done, tells every rank
// that the receive buffer of this epoch may be overwritten.
// all_out != 0: all-reduce mode, the reduced rows are also stored into every rank's gathered output buffer.
struct PeerOut {
    __nv_bfloat16* p[MAX_RANKS];
};
__global__ void __launch_bounds__(256) rs_reduce_kernel(const __nv_bfloat16* __restrict__ recv, __nv_bfloat16* __restrict__ out,
                                                        const __nv_bfloat16* __restrict__ bias,
                                                        const __nv_bfloat16* __restrict__ residual, int world, int rank,
                                                        int rows, int n, const uint32_t* ready_flags, uint32_t epoch,
                                                        PeerPads pads, int sig_offset, unsigned* counter, int all_out,
                                                        PeerOut gathered, const uint32_t* gfree_flags, uint32_t gfree_epoch,
                                                        int sig2_offset, int* status) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        int ok = 1;
        for (int src = 0; src < world && ok; ++src) {
            if (src == rank) continue;
            if (!wait_flag(ready_flags + src, epoch)) {
                atomicExch(status, 420 + src);
                ok = 0;
            }
            if (ok && all_out && !wait_flag(gfree_flags + src, gfree_epoch)) {
                atomicExch(status, 480 + src);
                ok = 0;
            }
        }
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    const size_t slot = (size_t)rows * n;
    const size_t nvec = slot / 8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int src = 0; src < world; ++src) {
            const uint4 v = *reinterpret_cast<const uint4*>(recv + src * slot + i * 8);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                acc[2 * t] += bf16_lo(w[t]);
                acc[2 * t + 1] += bf16_hi(w[t]);
            }
        }
        const size_t e = i * 8;
        if (bias) {
            const int col = (int)(e % n);
#pragma unroll
            for (int t = 0; t < 8; ++t) acc[t] += __bfloat162float(bias[col + t]);
        }
        if (residual) {
            const uint4 v = *reinterpret_cast<const uint4*>(residual + e);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                acc[2 * t] += bf16_lo(w[t]);
                acc[2 * t + 1] += bf16_hi(w[t]);
            }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        if (!all_out) {
            *reinterpret_cast<uint4*>(out + e) = o;
        } else {
            for (int dst = 0; dst < world; ++dst)
                *reinterpret_cast<uint4*>(gathered.p[dst] + (size_t)rank * slot + e) = o;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned old = atomicAdd(counter, 1u);
        if (old == gridDim.x - 1) {
            atomicExch(counter, 0u);
            __threadfence_system();
            for (int dst = 0; dst < world; ++dst) {
                st_release_sys(pads.p[dst] + sig_offset + rank, epoch);
                if (all_out) st_release_sys(pads.p[dst] + sig2_offset + rank, epoch);
            }
        }
    }
}

// All-reduce tail: wait until every rank has stored its reduced rows into this rank's gathered buffer, copy the buffer
// to the caller's tensor, then tell every rank this gathered buffer may be rewritten.
__global__ void __launch_bounds__(256) gathered_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nvec,
                                                            const uint32_t* ready_flags, uint32_t epoch, PeerPads pads,
                                                            int world, int rank, int sig_offset, unsigned* counter,
                                                            int* status) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        int ok = 1;
        for (int r = 0; r < world && ok; ++r)
            if (r != rank && !wait_flag(ready_flags + r, epoch)) {
                atomicExch(status, 500 + r);
                ok = 0;
            }
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = src[i];
    __syncthreads();
    if (threadIdx.x == 0) grid_done_signal(counter, pads.p, world, rank, sig_offset, epoch);
}

// Plain all-gather of published shards into a local tensor (for consumers that are not GEMMs).
__global__ void __launch_bounds__(256) symm_gather_kernel(PeerPads srcs, uint4* __restrict__ dst, size_t per_rank_vec,
                                                          const uint32_t* ready_flags, uint32_t epoch, PeerPads pads,
                                                          int world, int rank, int sig_offset, unsigned* counter,
                                                          int* status) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        int ok = 1;
        for (int r = 0; r < world && ok; ++r)
            if (r != rank && !wait_flag(ready_flags + r, epoch)) {
                atomicExch(status, 520 + r);
                ok = 0;
            }
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    const size_t total = per_rank_vec * world;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int src = (int)(i / per_rank_vec);
        const size_t off = i - (size_t)src * per_rank_vec;
        dst[i] = reinterpret_cast<const uint4*>(srcs.p[src])[off];
    }
    __syncthreads();
    if (threadIdx.x == 0 && sig_offset >= 0) grid_done_signal(counter, pads.p, world, rank, sig_offset, epoch);
}

// Release a gathered buffer: clear its block counters, then tell every rank (AG_DONE-style flag) that it may be
// overwritten.  Runs after the last local reader of the buffer, in stream order.
__global__ void __launch_bounds__(256) release_kernel(unsigned* cnt, int n, PeerPads pads, int world, int rank,
                                                      int sig_offset, uint32_t epoch) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) cnt[i] = 0u;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int dst = 0; dst < world; ++dst) st_release_sys(pads.p[dst] + sig_offset + rank, epoch);
    }
}

int copy_grid(size_t nvec) {
    size_t g = (nvec + 255) / 256;
    const size_t cap = (size_t)neox_sm_count() * 8;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace

// ------------------------------------------------------------------ symmetric memory plumbing (CUDA IPC)
// Symmetric buffers are plain device allocations exported to the other ranks of the node with CUDA IPC handles;
// python (parallel/symm_mem.py) exchanges the 64-byte handles through the process group.
extern "C" int neox_symm_alloc(void** out, unsigned long long bytes) {
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return NEOX_ERR_DRIVER;
    if (cudaMemset(p, 0, bytes) != cudaSuccess) return NEOX_ERR_DRIVER;
    if (cudaDeviceSynchronize() != cudaSuccess) return NEOX_ERR_DRIVER;
    *out = p;
    return 0;
}
extern "C" int neox_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : NEOX_ERR_DRIVER; }
extern "C" int neox_ipc_get_handle(void* p, void* handle64) {
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return NEOX_ERR_DRIVER;
    memcpy(handle64, &h, sizeof(h));
    return 0;
}
extern "C" int neox_ipc_open(const void* handle64, void** out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return NEOX_ERR_DRIVER;
    *out = p;
    return 0;
}
extern "C" int neox_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : NEOX_ERR_DRIVER; }

extern "C" int neox_symm_publish(const void* src, void* dst, void* dst2, unsigned long long bytes,
                                 const void* done_flags, unsigned need, const unsigned long long* pad_ptrs, int world,
                                 int rank, int sig_offset, unsigned epoch, void* counter, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if ((bytes % 16) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15) ||
        (reinterpret_cast<uintptr_t>(dst2) & 15))
        return NEOX_ERR_ALIGN;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    PeerPads pads;
    memset(&pads, 0, sizeof(pads));
    for (int i = 0; i < world; ++i) pads.p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
    const size_t nvec = bytes / 16;
    publish_kernel<<<copy_grid(nvec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), static_cast<uint4*>(dst2), nvec,
        static_cast<const uint32_t*>(done_flags), need, pads, world, rank, sig_offset, epoch,
        static_cast<unsigned*>(counter), status);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// The GEMM D = epilogue(op(A) op(B)) with an optional BROADCAST job and an optional PUSH of its output.
//   bc_src != NULL: this rank's shard ([rows_per_shard, row_bytes]) is copied into slot [rank] of every rank's
//       gathered buffer bc_dst_ptrs[dst], flagging finished 128-row blocks in bc_cnt_ptrs[dst] (bc_local_cnt: local
//       scratch of world * rows_per_shard / 128 zeroed words); the first store to dst waits for
//       bc_free_flags[dst] >= bc_free_epoch (dst has released the buffer).
//   a_dep / b_dep: A / B IS the local gathered buffer; loads wait for dep_cnt[block] != 0.
//   scatter: the output goes to recv_ptrs[owner] (slot = this rank) instead of D; bias / add (bf16) are added first.
//   sig*/sig2*: end-of-grid signals written into every rank's pad (offset < 0: none).
extern "C" int neox_comm_gemm(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                              long long ldd, int a_mn, int b_mn, int d_fp32, const void* bias, const void* add,
                              long long ldadd, int add_fp32, void* preact, long long ldpre, int act, int world, int rank,
                              const void* bc_src, const unsigned long long* bc_dst_ptrs,
                              const unsigned long long* bc_cnt_ptrs, void* bc_local_cnt, const void* bc_free_flags,
                              unsigned bc_free_epoch,
                              int rows_per_shard, long long row_bytes, const void* dep_cnt, int a_dep, int b_dep,
                              int scatter, int rows_per_rank, const unsigned long long* recv_ptrs,
                              const void* free_flags, unsigned free_epoch, const unsigned long long* pad_ptrs,
                              int sig_offset, unsigned sig_value, int sig2_offset, unsigned sig2_value, void* counter,
                              int n_copy, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8))
        return NEOX_ERR_ALIGN;
    const bool bcast = bc_src != nullptr;
    const bool dep = a_dep || b_dep;
    if ((bcast || dep) && ((rows_per_shard % 128) || rows_per_shard <= 0 || (row_bytes % 16))) return NEOX_ERR_SHAPE;
    if (bcast && ((reinterpret_cast<uintptr_t>(bc_src) & 15) || !bc_local_cnt)) return NEOX_ERR_ALIGN;
    if (dep && !dep_cnt) return NEOX_ERR_SHAPE;
    if (scatter && ((rows_per_rank % BM) || (N % 8) || rows_per_rank * world != M || (add && add_fp32)))
        return NEOX_ERR_SHAPE;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;

    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = neox_make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, BM);
    else rc = neox_make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK);
    if (rc) return rc;
    static int use_pair = -1;
    if (use_pair < 0) {
        const char* e = getenv("NEOX_COMM_GEMM_2CTA");
        use_pair = (e && e[0] == '0') ? 0 : 1;
    }
    // the pair form wants at least one 256 x 256 tile per pair of SMs' worth of work; tiny problems keep one CTA
    const bool pair = use_pair && (long long)((M + 255) / 256) * ((N + BN - 1) / BN) >= 8;
    if (!b_mn) rc = neox_make_tmap_bf16_2d(&tmB, B, K, N, ldb, BK, pair ? BN / 2 : BN);
    else rc = neox_make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK);
    if (rc) return rc;
    OutMaps outm;
    memset(&outm, 0, sizeof(outm));
    if (scatter) {
        for (int r = 0; r < world; ++r) {
            const char* base = reinterpret_cast<const char*>(recv_ptrs[r]) + (size_t)rank * rows_per_rank * N * 2;
            rc = neox_make_tmap_bf16_2d(&outm.m[r], base, N, rows_per_rank, N, 64, 32);
            if (rc) return rc;
        }
    }

    CommParams cp;
    memset(&cp, 0, sizeof(cp));
    GemmParams& p = cp.g;
    p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn;
    p.D = D; p.ldd = ldd; p.d_fp32 = d_fp32;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.add = add; p.ldadd = ldadd; p.add_fp32 = add_fp32;
    p.preact = static_cast<__nv_bfloat16*>(preact); p.ldpre = ldpre;
    p.aux = nullptr; p.ldaux = 0; p.act = act; p.alpha = 1.0f; p.status = status;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    bool vec = scatter ? true : (al16(D) && (ldd % 8 == 0));
    if (bias) vec = vec && al16(bias);
    if (add) vec = vec && al16(add) && (ldadd % 8 == 0);
    if (preact) vec = vec && al16(preact) && (ldpre % 8 == 0);
    if (scatter && !vec) return NEOX_ERR_ALIGN;
    p.vec_ok = vec ? 1 : 0;
    cp.world = world; cp.rank = rank;
    cp.bcast = bcast ? 1 : 0;
    if (bcast || dep) {
        cp.shard_bytes = (long long)rows_per_shard * row_bytes;
        cp.block_bytes = 128LL * row_bytes;
        cp.blocks_per_rank = rows_per_shard / 128;
        cp.pieces_per_block = (int)((cp.block_bytes + PIECE_BYTES - 1) / PIECE_BYTES);
        cp.rows_per_shard = rows_per_shard;
        cp.a_dep = a_dep; cp.b_dep = b_dep;
        cp.dep_cnt = static_cast<const unsigned*>(dep_cnt);
    }
    if (bcast) {
        cp.bc_src = static_cast<const uint4*>(bc_src);
        for (int r = 0; r < world; ++r) {
            cp.bc_dst[r] = reinterpret_cast<uint4*>(bc_dst_ptrs[r]);
            cp.bc_cnt[r] = reinterpret_cast<unsigned*>(bc_cnt_ptrs[r]);
        }
        cp.bc_local_cnt = static_cast<unsigned*>(bc_local_cnt);
        cp.bc_free_flags = static_cast<const uint32_t*>(bc_free_flags);
        cp.bc_free_epoch = bc_free_epoch;
    }
    cp.scatter = scatter; cp.rows_per_rank = rows_per_rank;
    cp.free_flags = static_cast<const uint32_t*>(free_flags); cp.free_epoch = free_epoch;
    cp.sig_offset = sig_offset; cp.sig_value = sig_value;
    cp.sig2_offset = sig2_offset; cp.sig2_value = sig2_value;
    cp.counter = static_cast<unsigned*>(counter);
    if (sig_offset >= 0 || sig2_offset >= 0)
        for (int r = 0; r < world; ++r) cp.peer_pad[r] = reinterpret_cast<uint32_t*>(pad_ptrs[r]);
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(comm_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 COMM_SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(comm_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 PAIR_SMEM_BYTES) != cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr_set = true;
    }
    const int tile_m = pair ? 2 * BM : BM;
    const int num_m = (M + tile_m - 1) / tile_m, num_n = (N + BN - 1) / BN;
    const int sms = neox_sm_count();
    const int per_tile = pair ? 2 : 1;                  // CTAs per tile-processing unit
    int grid = num_m * num_n * per_tile;
    if (grid > sms) grid = sms / per_tile * per_tile;
    if (bcast) {
        // the last n_copy CTAs of the grid copy instead of computing; all CTAs must be co-resident (one per SM)
        if (n_copy < 1) n_copy = 8;
        if (n_copy > sms / 2) n_copy = sms / 2;
        if (pair) n_copy = (n_copy + 1) & ~1;           // copy CTAs come in pairs too
        if (grid + n_copy > sms) grid = (sms - n_copy) / per_tile * per_tile;
        cp.n_copy = n_copy;
        grid += n_copy;
    }
    if (!pair) {
        comm_gemm_kernel<false><<<grid, COMM_THREADS, COMM_SMEM_BYTES, stream>>>(tmA, tmB, outm, cp);
        return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(COMM_THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, comm_gemm_kernel<true>, tmA, tmB, outm, cp) == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// Reduce the receive buffer of a scattered GEMM.  gathered_ptrs != NULL selects all-reduce mode (see the kernel).
extern "C" int neox_rs_reduce(const void* recv, void* out, const void* bias, const void* residual, int world, int rank,
                              int rows, int n, const void* ready_flags, unsigned epoch,
                              const unsigned long long* pad_ptrs, int sig_offset, void* counter,
                              const unsigned long long* gathered_ptrs, const void* gfree_flags, unsigned gfree_epoch,
                              int sig2_offset, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if (n % 8) return NEOX_ERR_SHAPE;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    PeerPads pads;
    PeerOut g;
    memset(&pads, 0, sizeof(pads));
    memset(&g, 0, sizeof(g));
    for (int i = 0; i < world; ++i) pads.p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
    if (gathered_ptrs)
        for (int i = 0; i < world; ++i) g.p[i] = reinterpret_cast<__nv_bfloat16*>(gathered_ptrs[i]);
    const size_t nvec = (size_t)rows * n / 8;
    rs_reduce_kernel<<<copy_grid(nvec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(recv), static_cast<__nv_bfloat16*>(out),
        static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(residual), world, rank, rows, n,
        static_cast<const uint32_t*>(ready_flags), epoch, pads, sig_offset, static_cast<unsigned*>(counter),
        gathered_ptrs ? 1 : 0, g, static_cast<const uint32_t*>(gfree_flags), gfree_epoch, sig2_offset, status);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

extern "C" int neox_gathered_copy(const void* src, void* dst, unsigned long long bytes, const void* ready_flags,
                                  unsigned epoch, const unsigned long long* pad_ptrs, int world, int rank,
                                  int sig_offset, void* counter, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if ((bytes % 16) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
        return NEOX_ERR_ALIGN;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    PeerPads pads;
    memset(&pads, 0, sizeof(pads));
    for (int i = 0; i < world; ++i) pads.p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
    const size_t nvec = bytes / 16;
    gathered_copy_kernel<<<copy_grid(nvec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), nvec, static_cast<const uint32_t*>(ready_flags), epoch,
        pads, world, rank, sig_offset, static_cast<unsigned*>(counter), status);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// dst[world][bytes_per_rank] = every rank's published shard (src_ptrs = the staging buffer as mapped here).
extern "C" int neox_symm_gather(const unsigned long long* src_ptrs, void* dst, unsigned long long bytes_per_rank,
                                const void* ready_flags, unsigned epoch, const unsigned long long* pad_ptrs, int world,
                                int rank, int sig_offset, void* counter, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if ((bytes_per_rank % 16) || (reinterpret_cast<uintptr_t>(dst) & 15)) return NEOX_ERR_ALIGN;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    PeerPads pads, srcs;
    memset(&pads, 0, sizeof(pads));
    memset(&srcs, 0, sizeof(srcs));
    for (int i = 0; i < world; ++i) {
        pads.p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
        srcs.p[i] = reinterpret_cast<uint32_t*>(src_ptrs[i]);
    }
    const size_t per = bytes_per_rank / 16;
    symm_gather_kernel<<<copy_grid(per * world), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        srcs, static_cast<uint4*>(dst), per, static_cast<const uint32_t*>(ready_flags), epoch, pads, world, rank,
        sig_offset, static_cast<unsigned*>(counter), status);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

extern "C" int neox_symm_release(void* cnt, int n, const unsigned long long* pad_ptrs, int world, int rank,
                                 int sig_offset, unsigned epoch, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    PeerPads pads;
    memset(&pads, 0, sizeof(pads));
    for (int i = 0; i < world; ++i) pads.p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
    release_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned*>(cnt), n, pads, world, rank,
                                                                      sig_offset, epoch);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// ------------------------------------------------------------------ variable-split all-to-all of rows (MoE)
namespace {

struct A2AParams {
    const uint4* src;                 // local send rows, grouped by destination rank
    uint4* dst[MAX_RANKS];            // every rank's receive buffer (peer-mapped)
    long long send_off[MAX_RANKS];    // first local row for destination d
    long long send_cnt[MAX_RANKS];    // rows for destination d
    long long recv_off[MAX_RANKS];    // row offset of this rank's block inside destination d's buffer
    int row_vec;                      // 16-byte vectors per row
    int world, rank;
    const uint32_t* free_flags;       // local pad: free_flags[d] >= free_epoch  <=>  d's buffer may be rewritten
    uint32_t free_epoch;
};

// One warp per row: 32 lanes x 16 bytes = 512-byte contiguous segments, which travel as full NVLink packets.
// Destinations are visited starting at rank + 1 so that at any time every rank receives from a different peer.
__global__ void __launch_bounds__(256) a2a_push_kernel(A2AParams ap, PeerPads pads, int sig_offset, uint32_t epoch,
                                                       unsigned* counter, int* status) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gw = (long long)blockIdx.x * 8 + warp, GW = (long long)gridDim.x * 8;
    bool ok = true;
    for (int i = 0; i < ap.world && ok; ++i) {
        const int d = (ap.rank + 1 + i) % ap.world;
        if (ap.send_cnt[d] == 0) continue;
        if (d != ap.rank) {
            int okf = 1;
            if (lane == 0) okf = wait_flag(ap.free_flags + d, ap.free_epoch) ? 1 : 0;
            okf = __shfl_sync(0xffffffffu, okf, 0);
            if (!okf) {
                if (lane == 0) atomicExch(status, 540 + d);
                ok = false;
                break;
            }
        }
        const uint4* s = ap.src + ap.send_off[d] * ap.row_vec;
        uint4* o = ap.dst[d] + ap.recv_off[d] * ap.row_vec;
        for (long long r = gw; r < ap.send_cnt[d]; r += GW)
            for (int v = lane; v < ap.row_vec; v += 32) o[r * ap.row_vec + v] = __ldg(s + r * ap.row_vec + v);
    }
    __syncthreads();
    if (threadIdx.x == 0) grid_done_signal(counter, pads.p, ap.world, ap.rank, sig_offset, epoch);
}

}  // namespace

// Push this rank's rows to their destination ranks' receive buffers and signal "epoch" to everyone.
// send_off / send_cnt / recv_off: world entries each (rows).  The receiver calls neox_gathered_copy with the matching
// ready / done flag offsets to wait for all sources and move the rows into an ordinary tensor.
extern "C" int neox_a2a_push(const void* src, const unsigned long long* dst_ptrs, const long long* send_off,
                             const long long* send_cnt, const long long* recv_off, int row_bytes, int world, int rank,
                             const void* free_flags, unsigned free_epoch, const unsigned long long* pad_ptrs,
                             int sig_offset, unsigned epoch, void* counter, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if ((row_bytes % 16) || (reinterpret_cast<uintptr_t>(src) & 15)) return NEOX_ERR_ALIGN;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    A2AParams ap;
    memset(&ap, 0, sizeof(ap));
    PeerPads pads;
    memset(&pads, 0, sizeof(pads));
    long long total = 0;
    for (int i = 0; i < world; ++i) {
        ap.dst[i] = reinterpret_cast<uint4*>(dst_ptrs[i]);
        ap.send_off[i] = send_off[i];
        ap.send_cnt[i] = send_cnt[i];
        ap.recv_off[i] = recv_off[i];
        pads.p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
        total += send_cnt[i];
    }
    ap.src = static_cast<const uint4*>(src);
    ap.row_vec = row_bytes / 16;
    ap.world = world; ap.rank = rank;
    ap.free_flags = static_cast<const uint32_t*>(free_flags);
    ap.free_epoch = free_epoch;
    long long grid = (total + 7) / 8;
    const long long cap = (long long)neox_sm_count() * 4;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    a2a_push_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(ap, pads, sig_offset, epoch,
                                                                                   static_cast<unsigned*>(counter),
                                                                                   status);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// Wait (bounded) until flags[r] >= epoch for every r != rank; a stream-ordered guard in front of kernels that write
// into peers' buffers without checking themselves.
namespace {
__global__ void wait_flags_kernel(const uint32_t* flags, uint32_t epoch, int world, int rank, int* status) {
    for (int r = threadIdx.x; r < world; r += blockDim.x)
        if (r != rank && !wait_flag(flags + r, epoch)) atomicExch(status, 560 + r);
}
}  // namespace

// The same with a limit of `rounds` spin periods (about two seconds each): for waits on ranks that are only loosely
// coupled to this one (data-parallel peers, which may be a host hiccup behind), in a one-warp kernel of their own so
// that nothing else is held up while it spins.
namespace {
__global__ void wait_flags_long_kernel(const uint32_t* flags, uint32_t epoch, int world, int rank, int rounds,
                                       int* status) {
    for (int r = threadIdx.x; r < world; r += blockDim.x) {
        if (r == rank) continue;
        bool ok = false;
        for (int i = 0; i < rounds && !ok; ++i) ok = wait_flag(flags + r, epoch);
        if (!ok) atomicExch(status, 580 + r);
    }
}
}  // namespace

extern "C" int neox_wait_flags_long(const void* flags, unsigned epoch, int world, int rank, int rounds, void* stream) {
    if (world > MAX_RANKS || world < 1 || rounds < 1 || rounds > 600) return NEOX_ERR_TOO_LARGE;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    wait_flags_long_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint32_t*>(flags), epoch,
                                                                             world, rank, rounds, status);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

extern "C" int neox_wait_flags(const void* flags, unsigned epoch, int world, int rank, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    wait_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint32_t*>(flags), epoch, world,
                                                                        rank, status);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// ------------------------------------------------------------------ ZeRO-1 gradient / parameter traffic over peer memory
// The flat fp32 gradient buffer and the flat 16-bit parameter buffer of a bucket live in symmetric memory.
//   reduce-scatter: every rank announces "my gradients of this bucket are final" (neox_symm_release with n = 0 on the
//     READY slot); the owner of a shard then READS that shard from every rank's buffer over NVLink, adds the copies
//     in rank order in fp32 (bit-identical on every run), scales, and writes its own copy -- one pass, no staging
//     buffer, the only NVLink traffic is the (world - 1) / world of the bucket that NCCL's ring also moves.  When
//     done it tells every rank (DONE slot) that their buffers may be rewritten.
//   all-gather: after the optimizer step the owner WRITES its updated 16-bit shard into every rank's parameter buffer
//     and raises the GATHERED slot; consumers put neox_wait_flags in front of the first kernel that reads the bucket.
// Reference counterpart: DeepSpeed ZeRO stage 1's NCCL reduce-scatter / all-gather of flattened buckets
// (driven from megatron/training.py of the reference through deepspeed.initialize).
namespace {

struct PeerF32 {
    const float* p[MAX_RANKS];
};
struct PeerVec {
    uint4* p[MAX_RANKS];
};

__global__ void __launch_bounds__(256) zero_reduce_scatter_kernel(PeerF32 src, float* __restrict__ out, size_t lo,
                                                                  size_t nvec, float scale,
                                                                  const uint32_t* ready_flags, uint32_t epoch,
                                                                  PeerPads pads, int world, int rank, int done_offset,
                                                                  unsigned* counter, int* status) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        int ok = 1;
        for (int r = 0; r < world && ok; ++r)
            if (r != rank && !wait_flag(ready_flags + r, epoch)) {
                atomicExch(status, 600 + r);
                ok = 0;
            }
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;      // nothing reduced, DONE never raised: the peers' bounded waits report it too
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < world; ++r) {
            const float4 v = reinterpret_cast<const float4*>(src.p[r] + lo)[i];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
        reinterpret_cast<float4*>(out + lo)[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) grid_done_signal(counter, pads.p, world, rank, done_offset, epoch);
}

__global__ void __launch_bounds__(256) zero_param_push_kernel(const uint4* __restrict__ src, PeerVec dst, size_t nvec,
                                                              PeerPads pads, int world, int rank, int sig_offset,
                                                              uint32_t epoch, unsigned* counter) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = src[i];
        for (int d = 1; d < world; ++d) {
            int r = rank + d;
            if (r >= world) r -= world;
            dst.p[r][i] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) grid_done_signal(counter, pads.p, world, rank, sig_offset, epoch);
}

}  // namespace

// grad_ptrs[r]: rank r's flat fp32 gradient buffer (peer-mapped); this rank's shard is elements [lo, lo + n),
// lo and n multiples of 4.  ready_flags: local pad slots [ready_offset ...]; counter: a zero-initialised local word.
extern "C" int neox_zero_reduce_scatter(const unsigned long long* grad_ptrs, unsigned long long lo, unsigned long long n,
                                        float scale, const void* ready_flags, unsigned epoch,
                                        const unsigned long long* pad_ptrs, int world, int rank, int done_offset,
                                        void* counter, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if ((lo % 4) || (n % 4)) return NEOX_ERR_ALIGN;
    if (n == 0) return 0;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    PeerF32 src;
    PeerPads pads;
    memset(&src, 0, sizeof(src));
    memset(&pads, 0, sizeof(pads));
    for (int i = 0; i < world; ++i) {
        src.p[i] = reinterpret_cast<const float*>(grad_ptrs[i]);
        pads.p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
    }
    const size_t nvec = n / 4;
    zero_reduce_scatter_kernel<<<copy_grid(nvec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, reinterpret_cast<float*>(grad_ptrs[rank]), lo, nvec, scale, static_cast<const uint32_t*>(ready_flags),
        epoch, pads, world, rank, done_offset, static_cast<unsigned*>(counter), status);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// param_ptrs[r]: rank r's flat parameter buffer (peer-mapped); copies `bytes` (a multiple of 16) starting at byte
// offset `byte_lo` of this rank's buffer to the same offset of every other rank's, then raises slot sig_offset.
extern "C" int neox_zero_param_push(const unsigned long long* param_ptrs, unsigned long long byte_lo,
                                    unsigned long long bytes, const unsigned long long* pad_ptrs, int world, int rank,
                                    int sig_offset, unsigned epoch, void* counter, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if ((byte_lo % 16) || (bytes % 16)) return NEOX_ERR_ALIGN;
    PeerVec dst;
    PeerPads pads;
    memset(&dst, 0, sizeof(dst));
    memset(&pads, 0, sizeof(pads));
    for (int i = 0; i < world; ++i) {
        dst.p[i] = reinterpret_cast<uint4*>(param_ptrs[i] + byte_lo);
        pads.p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
    }
    const size_t nvec = bytes / 16;
    zero_param_push_kernel<<<copy_grid(nvec > 0 ? nvec : 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4*>(param_ptrs[rank] + byte_lo), dst, nvec, pads, world, rank, sig_offset, epoch,
        static_cast<unsigned*>(counter));
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}
