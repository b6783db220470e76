// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a, tcgen05 + TMA).
//
// One kernel, same pipeline as gemm_sm100.cu (TMA ring -> tcgen05.mma -> TMEM -> epilogue warps), with two
// extensions that replace the NCCL calls around a column- / row-parallel linear layer:
//
//   * GATHERED OPERANDS (all-gather -> GEMM).  An operand whose rows are sharded over the tensor-parallel ranks is
//     described by one tensor map PER RANK, each over that rank's shard in peer-mapped ("symmetric") memory.  The
//     producer picks the map from the row coordinate, so every CTA fetches the remote tile it needs straight into its
//     own shared memory with a plain (non-multicast) TMA load: no gathered copy of the activation is ever written.
//     Before the first load from a peer the producer waits -- bounded -- for that peer's "shard is ready" flag; tiles
//     are visited local-shard-first so the wait overlaps useful work.  This covers the forward of a column-parallel
//     layer (A gathered along M), the data gradient of a row-parallel layer, and both weight gradients (the gathered
//     tensor is then the operand that is sharded along the contraction dimension).
//
//   * SCATTERED OUTPUT (GEMM -> reduce-scatter).  Row block m of the partial product belongs to rank m / rows_per_rank;
//     the epilogue stores each finished tile directly into the OWNER's receive buffer, slot [source rank], with
//     peer stores, so the transfer of tile i overlaps the math of tile i+1 (remote owners are served first).  A small
//     second kernel on the owner waits for every source's "all tiles pushed" flag and adds the slots in rank order in
//     fp32 (deterministic), fusing bias and residual.
//
// Flags are 32-bit epochs in the receiver's signal pad, written with st.release.sys after a system fence and read
// with ld.acquire.sys in a loop that gives up after ~2 s, records a status code and lets the kernel drain.
// No multicast of any kind is used.
#include "gemm_common.cuh"
#include "neox_b200.h"
#include <string.h>

using namespace gemm;

namespace {

constexpr int MAX_RANKS = 8;

struct CommMaps {
    CUtensorMap a[MAX_RANKS];
    CUtensorMap b[MAX_RANKS];
};

struct CommParams {
    GemmParams g;
    int world, rank;
    int a_split, b_split;            // rows of the operand's 2-D view owned by each rank (0 = operand is local)
    const uint32_t* gather_flags;     // local pad: gather_flags[src] >= gather_epoch  <=>  src's shard is published
    uint32_t gather_epoch;
    int scatter;                      // 1: epilogue pushes row blocks to their owner's receive buffer
    int rows_per_rank;                // scatter: output rows owned by each rank
    __nv_bfloat16* recv[MAX_RANKS];   // scatter: every rank's receive buffer [world][rows_per_rank][N]
    const uint32_t* free_flags;       // local pad: free_flags[owner] >= free_epoch  <=>  owner's buffer may be rewritten
    uint32_t free_epoch;
    uint32_t* peer_pad[MAX_RANKS];    // every rank's signal pad (peer-mapped)
    int sig_offset;                   // >= 0: when the whole grid is done, peer_pad[dst][sig_offset + rank] = sig_value
    uint32_t sig_value;
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

// Scatter epilogue for 32 columns of one row: partial = acc (+ bias) (+ local bf16 addend), stored as bf16 into the
// owner's receive slot (`dst` = start of this row in that slot).
__device__ __forceinline__ void push_chunk(const uint32_t (&r)[32], int row, int col0, const GemmParams& p,
                                           __nv_bfloat16* dst) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    if (p.vec_ok && col0 + 32 <= p.N) {
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
        uint4* o = reinterpret_cast<uint4*>(dst + col0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 q;
            q.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
            q.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
            q.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
            q.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
            o[j] = q;
        }
    } else {
        for (int i = 0; i < 32 && col0 + i < p.N; ++i) {
            float x = v[i];
            if (p.bias) x += __bfloat162float(p.bias[col0 + i]);
            if (p.add) x += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.add)[(long long)row * p.ldadd + col0 + i]);
            dst[col0 + i] = __float2bfloat16(x);
        }
    }
}

// Called by one thread per CTA after the CTA's last global / peer store (and a __syncthreads()).  The CTA that
// arrives last publishes `value` in slot [offset + rank] of every rank's signal pad.
__device__ __forceinline__ void grid_done_signal(unsigned* counter, uint32_t* const* pads, int world, int rank,
                                                 int offset, uint32_t value) {
    __threadfence_system();
    const unsigned old = atomicAdd(counter, 1u);
    if (old == gridDim.x - 1) {
        atomicExch(counter, 0u);
        __threadfence_system();
        for (int dst = 0; dst < world; ++dst) st_release_sys(pads[dst] + offset + rank, value);
    }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
comm_gemm_kernel(const __grid_constant__ CommMaps maps, const CommParams cp) {
    const GemmParams& p = cp.g;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* tfull = empty + STAGES;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 4);
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_m = (p.M + BM - 1) / BM;
    const int num_n = (p.N + BN - 1) / BN;
    const int ntiles = num_m * num_n;
    const int nk = (p.K + BK - 1) / BK;
    // Rotation of the row-block order: gathered-A kernels start on the local shard, scattering kernels start on the
    // block of the next rank (remote owners first, own block last).
    int m_rot = 0;
    if (cp.a_split > 0 && !p.a_mn) m_rot = (cp.rank * cp.a_split) / BM;
    if (cp.scatter) m_rot = (((cp.rank + 1) % cp.world) * cp.rows_per_rank) / BM;

    auto coords = [&](int tile, int& m_blk, int& n_blk) {
        tile_coords(tile, num_m, num_n, m_blk, n_blk);
        m_blk = (m_blk + m_rot) % num_m;
    };

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            uint32_t ready = 1u << cp.rank;      // bit r: rank r's shard is known to be ready
            auto need = [&](int src) -> bool {
                if (ready & (1u << src)) return true;
                if (!wait_flag(cp.gather_flags + src, cp.gather_epoch)) {
                    atomicExch(p.status, 400 + src);
                    return false;
                }
                // the shard was written through the generic proxy; TMA reads through the async proxy
                asm volatile("fence.proxy.async.global;" ::: "memory");
                ready |= 1u << src;
                return true;
            };
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                int m_blk, n_blk;
                coords(tile, m_blk, n_blk);
                for (int kb = 0; kb < nk && ok; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1)) {
                        atomicExch(p.status, 101);
                        ok = false;
                        break;
                    }
                    // y coordinate (row of the operand's 2-D view) decides which rank holds the tile
                    int ay = p.a_mn ? kb * BK : m_blk * BM;
                    int by = p.b_mn ? kb * BK : n_blk * BN;
                    int asrc = cp.rank, bsrc = cp.rank;
                    if (cp.a_split > 0) {
                        asrc = ay / cp.a_split;
                        ay -= asrc * cp.a_split;
                        if (asrc >= cp.world) asrc = cp.world - 1;
                    }
                    if (cp.b_split > 0) {
                        bsrc = by / cp.b_split;
                        by -= bsrc * cp.b_split;
                        if (bsrc >= cp.world) bsrc = cp.world - 1;
                    }
                    if (!need(asrc) || !need(bsrc)) {
                        ok = false;
                        break;
                    }
                    const CUtensorMap* ma = &maps.a[cp.a_split > 0 ? asrc : 0];
                    const CUtensorMap* mb = &maps.b[cp.b_split > 0 ? bsrc : 0];
                    mbar_expect_tx(&full[stage], A_STAGE_BYTES + B_STAGE_BYTES);
                    uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
                    uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
                    if (!p.a_mn) {
                        tma_load_2d(a_dst, ma, &full[stage], kb * BK, ay);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_2d(a_dst + j * (64 * BK * 2), ma, &full[stage], m_blk * BM + j * 64, ay);
                    }
                    if (!p.b_mn) {
                        tma_load_2d(b_dst, mb, &full[stage], kb * BK, by);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(b_dst + j * (64 * BK * 2), mb, &full[stage], n_blk * BN + j * 64, by);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn, p.b_mn);
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t bphase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
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
                    const uint32_t a_base = smem_u32(sA + stage * A_STAGE_BYTES);
                    const uint32_t b_base = smem_u32(sB + stage * B_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t adesc = p.a_mn ? make_smem_desc_sw128(a_base + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                                      : make_smem_desc_sw128(a_base + k * (UMMA_K * 2), 16, 1024);
                        const uint64_t bdesc = p.b_mn ? make_smem_desc_sw128(b_base + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                                      : make_smem_desc_sw128(b_base + k * (UMMA_K * 2), 16, 1024);
                        umma_bf16_ss(tmem_d, adesc, bdesc, idesc, (kb | k) != 0);
                    }
                    umma_commit(&empty[stage]);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(&tfull[buf]);
                buf ^= 1;
                if (buf == 0) bphase ^= 1;
            }
        }
    } else {
        const int q = warp & 3;
        int buf = 0;
        uint32_t bphase = 0;
        uint32_t freed = 1u << cp.rank;   // bit o: owner o's receive buffer is known to be reusable
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            int m_blk, n_blk;
            coords(tile, m_blk, n_blk);
            if (!mbar_wait_warp(&tfull[buf], bphase)) {
                if (lane == 0) atomicExch(p.status, 104);
                break;
            }
            tc_fence_after();
            const int row = m_blk * BM + q * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
            // scatter mode: this row lives in the receive buffer of its owner, slot = my rank
            __nv_bfloat16* push = nullptr;
            if (cp.scatter) {
                const int owner = min((m_blk * BM) / cp.rows_per_rank, cp.world - 1);   // warp-uniform
                if (!(freed & (1u << owner))) {
                    int ok = 1;
                    if (lane == 0) ok = wait_flag(cp.free_flags + owner, cp.free_epoch) ? 1 : 0;
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) {
                        if (lane == 0) atomicExch(p.status, 440 + owner);
                        break;
                    }
                    freed |= 1u << owner;
                }
                const int lrow = row - owner * cp.rows_per_rank;
                push = cp.recv[owner] + ((size_t)cp.rank * cp.rows_per_rank + lrow) * (size_t)p.N;
            }
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int col0 = n_blk * BN + c * 32;
                if (col0 >= p.N) break;
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_wait_ld();
                if (row < p.M) {
                    if (!cp.scatter) {
                        epilogue_chunk(r, row, col0, p);
                    } else {
                        push_chunk(r, row, col0, p, push);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[buf]);
            buf ^= 1;
            if (buf == 0) bphase ^= 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && cp.sig_offset >= 0) grid_done_signal(cp.counter, cp.peer_pad, cp.world, cp.rank, cp.sig_offset, cp.sig_value);
}

// Copy this rank's shard into its symmetric staging buffer and tell every rank it is there.
//   wait  : the buffer was last read by the peers' GEMMs of epoch `need`; done_flags[peer] >= need says they finished
//   copy  : 16-byte vectors, grid-stride
//   signal: last CTA writes `epoch` into slot [sig_offset + rank] of every pad
__global__ void __launch_bounds__(256) publish_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nvec,
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
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = src[i];
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

extern "C" int neox_symm_publish(const void* src, void* dst, unsigned long long bytes, const void* done_flags,
                                 unsigned need, const unsigned long long* pad_ptrs, int world, int rank,
                                 int sig_offset, unsigned epoch, void* counter, void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if ((bytes % 16) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
        return NEOX_ERR_ALIGN;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    PeerPads pads;
    memset(&pads, 0, sizeof(pads));
    for (int i = 0; i < world; ++i) pads.p[i] = reinterpret_cast<uint32_t*>(pad_ptrs[i]);
    const size_t nvec = bytes / 16;
    publish_kernel<<<copy_grid(nvec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), nvec, static_cast<const uint32_t*>(done_flags), need,
        pads, world, rank, sig_offset, epoch, static_cast<unsigned*>(counter), status);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
}

// a_ptrs / b_ptrs: per-rank base pointers of the operand (only index 0 is read when the operand is local).
// a_split / b_split: rows of the operand's 2-D view held by EACH rank (0 = local operand).
extern "C" int neox_comm_gemm(const unsigned long long* a_ptrs, const unsigned long long* b_ptrs, void* D, int M,
                              int N, int K, long long lda, long long ldb, long long ldd, int a_mn, int b_mn,
                              int d_fp32, const void* bias, const void* add, long long ldadd, int add_fp32,
                              void* preact, long long ldpre, int act, int world, int rank, int a_split, int b_split,
                              const void* gather_flags, unsigned gather_epoch, int scatter, int rows_per_rank,
                              const unsigned long long* recv_ptrs, const void* free_flags, unsigned free_epoch,
                              const unsigned long long* pad_ptrs, int sig_offset, unsigned sig_value, void* counter,
                              void* stream) {
    if (world > MAX_RANKS || world < 1) return NEOX_ERR_TOO_LARGE;
    if ((lda % 8) || (ldb % 8)) return NEOX_ERR_ALIGN;
    if (a_split > 0 && (a_split % (a_mn ? BK : BM))) return NEOX_ERR_SHAPE;
    if (b_split > 0 && (b_split % (b_mn ? BK : BN))) return NEOX_ERR_SHAPE;
    if (scatter && ((rows_per_rank % BM) || (N % 8) || rows_per_rank * world != M || (add && add_fp32)))
        return NEOX_ERR_SHAPE;
    int* status = neox_status_word();
    if (!status) return NEOX_ERR_DRIVER;
    CommMaps maps;
    memset(&maps, 0, sizeof(maps));
    const int na = a_split > 0 ? world : 1, nb = b_split > 0 ? world : 1;
    for (int r = 0; r < na; ++r) {
        const void* ptr = reinterpret_cast<const void*>(a_ptrs[r]);
        // K-major: dims {K, rows}, box {BK, BM};  MN-major: dims {M, k-rows}, box {64, BK}
        const unsigned long long rows = a_split > 0 ? (unsigned long long)a_split : (unsigned long long)(a_mn ? K : M);
        int rc = a_mn ? neox_make_tmap_bf16_2d(&maps.a[r], ptr, M, rows, lda, 64, BK)
                      : neox_make_tmap_bf16_2d(&maps.a[r], ptr, K, rows, lda, BK, BM);
        if (rc) return rc;
    }
    for (int r = 0; r < nb; ++r) {
        const void* ptr = reinterpret_cast<const void*>(b_ptrs[r]);
        const unsigned long long rows = b_split > 0 ? (unsigned long long)b_split : (unsigned long long)(b_mn ? K : N);
        int rc = b_mn ? neox_make_tmap_bf16_2d(&maps.b[r], ptr, N, rows, ldb, 64, BK)
                      : neox_make_tmap_bf16_2d(&maps.b[r], ptr, K, rows, ldb, BK, BN);
        if (rc) return rc;
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
    p.vec_ok = vec ? 1 : 0;
    cp.world = world; cp.rank = rank; cp.a_split = a_split; cp.b_split = b_split;
    cp.gather_flags = static_cast<const uint32_t*>(gather_flags); cp.gather_epoch = gather_epoch;
    cp.scatter = scatter; cp.rows_per_rank = rows_per_rank;
    cp.free_flags = static_cast<const uint32_t*>(free_flags); cp.free_epoch = free_epoch;
    if (scatter)
        for (int r = 0; r < world; ++r) cp.recv[r] = reinterpret_cast<__nv_bfloat16*>(recv_ptrs[r]);
    cp.sig_offset = sig_offset; cp.sig_value = sig_value; cp.counter = static_cast<unsigned*>(counter);
    if (sig_offset >= 0)
        for (int r = 0; r < world; ++r) cp.peer_pad[r] = reinterpret_cast<uint32_t*>(pad_ptrs[r]);
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(comm_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return NEOX_ERR_LAUNCH;
        attr_set = true;
    }
    const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
    int grid = num_m * num_n;
    const int sms = neox_sm_count();
    if (grid > sms) grid = sms;
    comm_gemm_kernel<<<grid, NUM_THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(maps, cp);
    return cudaGetLastError() == cudaSuccess ? 0 : NEOX_ERR_LAUNCH;
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
