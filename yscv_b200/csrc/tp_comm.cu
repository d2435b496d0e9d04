// Exchange regions for tensor-parallel decode steps.
//
// The reference has no multi-GPU inference path (crates/yscv-model/src/distributed.rs:27
// says so; its collectives are byte-level TCP for training). Here one process drives one GPU;
// a rank allocates an exchange region in its own HBM, exports it with CUDA IPC, and maps every
// peer's region, so that the decode-step kernel of a rank can store its partial sums straight
// into the peers' memory over NVLink (plain peer stores; no multicast, no collective library)
// and poll its own region for theirs. The handles travel between the processes by whatever
// the host uses for rendezvous (the Python side uses torch.distributed's all_gather).
#include <cstring>

#include "common.cuh"

using namespace yscv;

namespace {
size_t region_bytes(int world, size_t cap_rows) {
    // [2 parities][world sources][cap_rows] partial-sum words + [2][world][2] greedy-token words
    return ((size_t)2 * world * cap_rows + (size_t)2 * world * 2) * sizeof(unsigned long long);
}
}  // namespace

extern "C" {

int yscv_cuda_tp_comm_create(yscv_cuda_ctx *ctx, int rank, int world, size_t max_rows,
                             yscv_cuda_tp_comm **out, uint8_t handle_out[YSCV_CUDA_TP_HANDLE_BYTES]) {
    if (!ctx || !out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    if (world < 2 || world > 8 || rank < 0 || rank >= world)
        return fail(YSCV_CUDA_ERR_BAD_ARG, "rank %d of %d: a tensor-parallel group has 2 to 8 ranks", rank, world);
    if (max_rows == 0 || max_rows > (1u << 20)) return fail(YSCV_CUDA_ERR_BAD_ARG, "max_rows=%zu", max_rows);
    static_assert(sizeof(cudaIpcMemHandle_t) <= YSCV_CUDA_TP_HANDLE_BYTES, "IPC handle does not fit");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    auto *c = new yscv_cuda_tp_comm();
    c->device = ctx->device;
    c->rank = rank;
    c->world = world;
    c->cap_rows = max_rows;
    c->bytes = region_bytes(world, max_rows);
    cudaError_t e = cudaMalloc(&c->local, c->bytes);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, c->bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&c->d_seq), sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(c->d_seq, 0, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (c->local) cudaFree(c->local);
        if (c->d_seq) cudaFree(c->d_seq);
        delete c;
        return fail(YSCV_CUDA_ERR_CUDA, "exchange region: %s", cudaGetErrorString(e));
    }
    c->peer[rank] = c->local;
    if (handle_out) {
        memset(handle_out, 0, YSCV_CUDA_TP_HANDLE_BYTES);
        cudaIpcMemHandle_t h;
        e = cudaIpcGetMemHandle(&h, c->local);
        if (e != cudaSuccess) {
            cudaFree(c->local);
            cudaFree(c->d_seq);
            delete c;
            return fail(YSCV_CUDA_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
        }
        memcpy(handle_out, &h, sizeof(h));
    }
    *out = c;
    return YSCV_CUDA_OK;
}

int yscv_cuda_tp_comm_connect(yscv_cuda_tp_comm *comm, const uint8_t *handles) {
    if (!comm || !handles) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (comm->connected) return fail(YSCV_CUDA_ERR_BAD_ARG, "already connected");
    YSCV_CUDA_TRY(cudaSetDevice(comm->device));
    for (int r = 0; r < comm->world; ++r) {
        if (r == comm->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * YSCV_CUDA_TP_HANDLE_BYTES, sizeof(h));
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < r; ++q)
                if (comm->opened[q]) { cudaIpcCloseMemHandle(comm->peer[q]); comm->opened[q] = false; comm->peer[q] = nullptr; }
            return fail(YSCV_CUDA_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d): %s", r, cudaGetErrorString(e));
        }
        comm->peer[r] = p;
        comm->opened[r] = true;
    }
    comm->connected = true;
    return YSCV_CUDA_OK;
}

int yscv_cuda_tp_comm_connect_unanswered(yscv_cuda_tp_comm *comm) {
    if (!comm) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (comm->connected) return fail(YSCV_CUDA_ERR_BAD_ARG, "already connected");
    YSCV_CUDA_TRY(cudaSetDevice(comm->device));
    YSCV_CUDA_TRY(cudaMalloc(&comm->standin, comm->bytes * (size_t)(comm->world - 1)));
    YSCV_CUDA_TRY(cudaMemset(comm->standin, 0, comm->bytes * (size_t)(comm->world - 1)));
    int j = 0;
    for (int r = 0; r < comm->world; ++r) {
        if (r == comm->rank) continue;
        comm->peer[r] = static_cast<char *>(comm->standin) + (size_t)(j++) * comm->bytes;
    }
    comm->connected = true;
    return YSCV_CUDA_OK;
}

void yscv_cuda_tp_comm_destroy(yscv_cuda_tp_comm *comm) {
    if (!comm) return;
    cudaSetDevice(comm->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < comm->world; ++r)
        if (comm->opened[r]) cudaIpcCloseMemHandle(comm->peer[r]);
    if (comm->standin) cudaFree(comm->standin);
    if (comm->local) cudaFree(comm->local);
    if (comm->d_seq) cudaFree(comm->d_seq);
    delete comm;
}

}  // extern "C"
