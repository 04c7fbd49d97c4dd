// The one exchange step of the path inside the library: communicator, symmetric (peer-mapped) buffers, a
// cross-GPU barrier and the two forms of the column-split GEMM, for hosts that run one process per GPU.
//
// The reference has no distributed code (hgemm.zig:396-423 spawns threads only); the arithmetic per column
// block is md_hgemm_nn / md_hgemm_nt.  What this file adds around it:
//   * md_comm_init        an NCCL communicator from a unique id the caller distributes (rank 0 makes it with
//                         md_comm_unique_id and ships the 128 bytes however it likes).  NCCL is resolved at run
//                         time (dlopen of libnccl.so.2), so the library loads on machines without it and a process
//                         that already carries an NCCL (e.g. through PyTorch) shares that copy.
//   * md_comm_symm_alloc  a buffer of the same size on every rank, mapped into every other rank through CUDA IPC
//                         (handles all-gathered over the communicator), so kernels can store into the peers' copies.
//   * md_comm_barrier     a one-CTA kernel: release-store an epoch into every peer's signal pad, wait (bounded) for
//                         every peer's epoch in the own pad.  Stream-ordered, no host round trip.
//   * md_hgemm_colsplit_allgather   baseline: tcgen05 GEMM into a contiguous [M, N/world] block, ncclAllGather,
//                         one re-layout kernel into [M, N].
//   * md_hgemm_colsplit_fused       the GEMM whose push warps store every finished tile into all peers' C
//                         (md_hgemm_colsplit_push) between two barriers; no collective, no re-layout.
// No load ever targets peer memory (only plain stores and the barrier's flag loads of the own pad).
#include "md_internal.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

namespace {

constexpr int COMM_MAX_WORLD = 8;
constexpr int PAD_CHANNELS = 4;
constexpr unsigned long long BARRIER_BUDGET_NS = 2000000000ull;  // 2 s: covers a peer that is still computing

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi g_nccl;

int nccl_load(md_ctx* ctx) {
    if (g_nccl.lib) return MD_OK;
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return md_fail(ctx, MD_ERR_NCCL, "NCCL is not available: %s", dlerror());
    NcclApi api;
    api.lib = lib;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(lib, "ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather || !api.GetErrorString)
        return md_fail(ctx, MD_ERR_NCCL, "libnccl lacks one of the five entry points this library uses");
    g_nccl = api;
    return MD_OK;
}

#define MD_NCCL(ctx, expr)                                                                            \
    do {                                                                                              \
        ncclResult_t _r = (expr);                                                                     \
        if (_r != ncclSuccess)                                                                        \
            return md_fail((ctx), MD_ERR_NCCL, "%s failed: %s", #expr, g_nccl.GetErrorString(_r));    \
    } while (0)

struct PeerPads {
    unsigned* pad[COMM_MAX_WORLD];
};

// One thread per peer: tell the peer this rank has arrived at `epoch`, then wait until the peer has.  The epochs
// only grow (wrap-safe comparison), so a pad needs no clearing between barriers.
__global__ void comm_barrier_kernel(PeerPads pads, int rank, int world, int channel, unsigned epoch, md_devflags* flags) {
    const int t = threadIdx.x;
    if (t >= world || t == rank) return;
    __threadfence_system();  // everything this GPU stored before the barrier is performed first
    unsigned* theirs = pads.pad[t] + channel * COMM_MAX_WORLD + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    const unsigned* mine = pads.pad[rank] + channel * COMM_MAX_WORLD + t;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned spin = 0;; ++spin) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int)(v - epoch) >= 0) return;
        if ((spin & 255u) == 255u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - t0 > BARRIER_BUDGET_NS) {
                md_flag_timeout(flags, 200u + (unsigned)t);  // site 200 + peer: that peer never arrived
                return;
            }
        }
        __nanosleep(100);
    }
}

// gathered [world][M][n] -> c [M][world * n], 16 bytes per thread (n % 8 == 0).
__global__ void __launch_bounds__(256)
gather_colblocks_kernel(const uint4* __restrict__ gathered, uint4* __restrict__ c, int world, long long M, int n8) {
    const long long total = (long long)world * M * n8;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int col = (int)(i % n8);
        const long long row = (i / n8) % M;
        const int g = (int)(i / ((long long)n8 * M));
        c[(row * world + g) * n8 + col] = gathered[i];
    }
}

}  // namespace

struct md_comm {
    md_ctx* ctx = nullptr;
    int rank = 0, world = 1;
    ncclComm_t nccl = nullptr;
    struct Symm {
        void* local = nullptr;
        size_t bytes = 0;
        void* peer[COMM_MAX_WORLD] = {};  // peer[rank] == local
    };
    std::vector<Symm> symm;
    unsigned* pad = nullptr;  // symmetric signal pad: [PAD_CHANNELS][COMM_MAX_WORLD] epochs
    PeerPads pads = {};
    unsigned epoch[PAD_CHANNELS] = {};
    void* handle_stage = nullptr;  // device staging for the IPC handle exchange
    void* block = nullptr;         // all-gather baseline: this rank's contiguous block and the gathered blocks
    void* gathered = nullptr;
    size_t block_cap = 0, gathered_cap = 0;
};

namespace {

int symm_alloc(md_comm* comm, size_t bytes, md_comm::Symm* out) {
    md_ctx* ctx = comm->ctx;
    md_comm::Symm s;
    s.bytes = bytes;
    MD_CUDA(ctx, cudaMalloc(&s.local, bytes ? bytes : 1));
    MD_CUDA(ctx, cudaMemsetAsync(s.local, 0, bytes, ctx->stream));
    s.peer[comm->rank] = s.local;
    if (comm->world > 1) {
        cudaIpcMemHandle_t mine, all[COMM_MAX_WORLD];
        MD_CUDA(ctx, cudaIpcGetMemHandle(&mine, s.local));
        char* stage = static_cast<char*>(comm->handle_stage);
        MD_CUDA(ctx, cudaMemcpyAsync(stage + comm->rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice,
                                     ctx->stream));
        // the memset above precedes this collective on the stream: a peer that receives the handle finds zeros
        MD_NCCL(ctx, g_nccl.AllGather(stage + comm->rank * sizeof(mine), stage, sizeof(mine), ncclChar, comm->nccl,
                                      ctx->stream));
        MD_CUDA(ctx, cudaMemcpyAsync(all, stage, sizeof(mine) * comm->world, cudaMemcpyDeviceToHost, ctx->stream));
        MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        for (int r = 0; r < comm->world; ++r) {
            if (r == comm->rank) continue;
            MD_CUDA(ctx, cudaIpcOpenMemHandle(&s.peer[r], all[r], cudaIpcMemLazyEnablePeerAccess));
        }
    } else {
        MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    *out = s;
    return MD_OK;
}

void symm_release(md_comm* comm, md_comm::Symm& s) {
    for (int r = 0; r < comm->world; ++r)
        if (r != comm->rank && s.peer[r]) cudaIpcCloseMemHandle(s.peer[r]);
    if (s.local) cudaFree(s.local);
    s = md_comm::Symm();
}

int barrier(md_comm* comm, int channel) {
    md_ctx* ctx = comm->ctx;
    if (comm->world == 1) return MD_OK;
    const unsigned epoch = ++comm->epoch[channel];
    comm_barrier_kernel<<<1, 32, 0, ctx->stream>>>(comm->pads, comm->rank, comm->world, channel, epoch, ctx->flags);
    MD_LAUNCH_CHECK(ctx, "comm_barrier_kernel");
    return MD_OK;
}

}  // namespace

#define MD_NEED_COMM(comm) \
    do { if (!(comm) || !(comm)->ctx) return MD_ERR_INVALID_ARG; } while (0)

extern "C" {

int md_comm_unique_id(md_ctx* ctx, void* id_out) {
    if (!ctx) return MD_ERR_INVALID_ARG;
    if (!id_out) return md_fail(ctx, MD_ERR_INVALID_ARG, "md_comm_unique_id: null output");
    MD_TRY(nccl_load(ctx));
    ncclUniqueId id;
    MD_NCCL(ctx, g_nccl.GetUniqueId(&id));
    static_assert(sizeof(id) == MD_COMM_ID_BYTES, "unique id size");
    memcpy(id_out, &id, sizeof(id));
    return MD_OK;
}

int md_comm_init(md_ctx* ctx, const void* unique_id, int rank, int world, md_comm** out) {
    if (!ctx) return MD_ERR_INVALID_ARG;
    if (!out || !unique_id) return md_fail(ctx, MD_ERR_INVALID_ARG, "md_comm_init: null argument");
    *out = nullptr;
    if (world < 1 || world > COMM_MAX_WORLD || rank < 0 || rank >= world)
        return md_fail(ctx, MD_ERR_INVALID_ARG, "md_comm_init: rank %d of %d (1..%d ranks)", rank, world, COMM_MAX_WORLD);
    MD_CUDA(ctx, cudaSetDevice(ctx->device));
    md_comm* comm = new md_comm();
    comm->ctx = ctx;
    comm->rank = rank;
    comm->world = world;
    auto fail = [&](int st) {
        md_comm_destroy(comm);
        return st;
    };
    if (world > 1) {
        int st = nccl_load(ctx);
        if (st != MD_OK) return fail(st);
        ncclUniqueId id;
        memcpy(&id, unique_id, sizeof(id));
        const ncclResult_t r = g_nccl.CommInitRank(&comm->nccl, world, id, rank);
        if (r != ncclSuccess)
            return fail(md_fail(ctx, MD_ERR_NCCL, "ncclCommInitRank failed: %s", g_nccl.GetErrorString(r)));
        if (cudaMalloc(&comm->handle_stage, sizeof(cudaIpcMemHandle_t) * COMM_MAX_WORLD) != cudaSuccess)
            return fail(md_fail(ctx, MD_ERR_OOM, "md_comm_init: staging allocation failed"));
    }
    md_comm::Symm pad;
    int st = symm_alloc(comm, PAD_CHANNELS * COMM_MAX_WORLD * sizeof(unsigned), &pad);
    if (st != MD_OK) return fail(st);
    comm->symm.push_back(pad);
    comm->pad = static_cast<unsigned*>(pad.local);
    for (int r = 0; r < world; ++r) comm->pads.pad[r] = static_cast<unsigned*>(pad.peer[r]);
    *out = comm;
    return MD_OK;
}

int md_comm_destroy(md_comm* comm) {
    if (!comm) return MD_OK;
    md_ctx* ctx = comm->ctx;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& s : comm->symm) symm_release(comm, s);
    if (comm->handle_stage) cudaFree(comm->handle_stage);
    if (comm->block) cudaFree(comm->block);
    if (comm->gathered) cudaFree(comm->gathered);
    if (comm->nccl) g_nccl.CommDestroy(comm->nccl);
    delete comm;
    return MD_OK;
}

int md_comm_symm_alloc(md_comm* comm, size_t bytes, void** local_out) {
    MD_NEED_COMM(comm);
    md_ctx* ctx = comm->ctx;
    if (!local_out || bytes == 0) return md_fail(ctx, MD_ERR_INVALID_ARG, "md_comm_symm_alloc: null output or zero size");
    md_comm::Symm s;
    MD_TRY(symm_alloc(comm, bytes, &s));
    comm->symm.push_back(s);
    *local_out = s.local;
    return MD_OK;
}

int md_comm_symm_free(md_comm* comm, void* local) {
    MD_NEED_COMM(comm);
    md_ctx* ctx = comm->ctx;
    for (size_t i = 1; i < comm->symm.size(); ++i) {  // entry 0 is the signal pad
        if (comm->symm[i].local == local) {
            MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            symm_release(comm, comm->symm[i]);
            comm->symm.erase(comm->symm.begin() + i);
            return MD_OK;
        }
    }
    return md_fail(ctx, MD_ERR_INVALID_ARG, "md_comm_symm_free: not a buffer of this communicator");
}

int md_comm_barrier(md_comm* comm) {
    MD_NEED_COMM(comm);
    return barrier(comm, 2);
}

int md_hgemm_colsplit_fused(md_comm* comm, const uint16_t* a, const uint16_t* b_slice, uint16_t* c_symm, size_t M,
                            size_t N_total, size_t K, int b_layout) {
    MD_NEED_COMM(comm);
    md_ctx* ctx = comm->ctx;
    if (!a || !b_slice || !c_symm) return md_fail(ctx, MD_ERR_INVALID_ARG, "colsplit_fused: null tensor pointer");
    const size_t world = (size_t)comm->world;
    if (N_total % world || (N_total / world) % 8)
        return md_fail(ctx, MD_ERR_SHAPE, "colsplit_fused: N = %zu does not split into %zu blocks of a multiple of 8 columns",
                       N_total, world);
    const md_comm::Symm* s = nullptr;
    for (size_t i = 1; i < comm->symm.size(); ++i)
        if (comm->symm[i].local == c_symm) s = &comm->symm[i];
    if (!s) return md_fail(ctx, MD_ERR_INVALID_ARG, "colsplit_fused: C must come from md_comm_symm_alloc of this communicator");
    if (s->bytes < M * N_total * 2) return md_fail(ctx, MD_ERR_SHAPE, "colsplit_fused: the symmetric buffer is smaller than C");
    uint16_t* peers[COMM_MAX_WORLD];
    size_t np = 0;
    for (int r = 0; r < comm->world; ++r)
        if (r != comm->rank) peers[np++] = static_cast<uint16_t*>(s->peer[r]);
    const size_t n_local = N_total / world;
    MD_TRY(barrier(comm, 0));  // nobody still reads the previous contents of C
    MD_TRY(md_hgemm_colsplit_push(ctx, a, b_slice, c_symm, M, n_local, K, b_layout, N_total, comm->rank * n_local, np, peers));
    return barrier(comm, 1);   // every rank's pushes have landed
}

int md_hgemm_colsplit_allgather(md_comm* comm, const uint16_t* a, const uint16_t* b_slice, uint16_t* c_full, size_t M,
                                size_t N_total, size_t K, int b_layout) {
    MD_NEED_COMM(comm);
    md_ctx* ctx = comm->ctx;
    if (!a || !b_slice || !c_full) return md_fail(ctx, MD_ERR_INVALID_ARG, "colsplit_allgather: null tensor pointer");
    if (b_layout != 0 && b_layout != 1) return md_fail(ctx, MD_ERR_INVALID_ARG, "colsplit_allgather: b_layout must be 0 or 1");
    const size_t world = (size_t)comm->world;
    if (N_total % world || (N_total / world) % 8)
        return md_fail(ctx, MD_ERR_SHAPE,
                       "colsplit_allgather: N = %zu does not split into %zu blocks of a multiple of 8 columns", N_total, world);
    if (!md_is_device_ptr(a) || !md_is_device_ptr(b_slice) || !md_is_device_ptr(c_full))
        return md_fail(ctx, MD_ERR_UNSUPPORTED, "colsplit_allgather: device pointers only");
    const size_t n_local = N_total / world;
    if (M == 0 || n_local == 0) return MD_OK;
    if (world == 1) return b_layout == 0 ? md_hgemm_nn(ctx, a, b_slice, c_full, M, N_total, K)
                                         : md_hgemm_nt(ctx, a, b_slice, c_full, M, N_total, K);
    const size_t block_bytes = M * n_local * 2;
    auto grow = [&](void** p, size_t* cap, size_t need) -> int {
        if (*cap >= need) return MD_OK;
        if (ctx->capturing) return md_fail(ctx, MD_ERR_UNSUPPORTED, "colsplit_allgather: run the call once before capturing");
        if (*p) {
            MD_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            MD_CUDA(ctx, cudaFree(*p));
            *p = nullptr;
            *cap = 0;
        }
        MD_CUDA(ctx, cudaMalloc(p, need));
        *cap = need;
        return MD_OK;
    };
    MD_TRY(grow(&comm->block, &comm->block_cap, block_bytes));
    MD_TRY(grow(&comm->gathered, &comm->gathered_cap, block_bytes * world));
    uint16_t* block = static_cast<uint16_t*>(comm->block);
    MD_TRY(b_layout == 0 ? md_hgemm_nn(ctx, a, b_slice, block, M, n_local, K) : md_hgemm_nt(ctx, a, b_slice, block, M, n_local, K));
    MD_NCCL(ctx, g_nccl.AllGather(block, comm->gathered, M * n_local, ncclHalf, comm->nccl, ctx->stream));
    return md_gather_colblocks(ctx, static_cast<const uint16_t*>(comm->gathered), c_full, world, M, n_local);
}

}  // extern "C"

// The re-layout of the all-gather baseline as one kernel (md_gather_colblocks in md_api.cu calls it when the
// blocks are 16-byte addressable).
int md_launch_gather_colblocks(md_ctx* ctx, const uint16_t* gathered, uint16_t* c, size_t world, size_t M, size_t n_local) {
    const long long total = (long long)world * M * (n_local / 8);
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    gather_colblocks_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const uint4*>(gathered), reinterpret_cast<uint4*>(c),
                                                           (int)world, (long long)M, (int)(n_local / 8));
    MD_LAUNCH_CHECK(ctx, "gather_colblocks_kernel");
    return MD_OK;
}
