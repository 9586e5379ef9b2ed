// The multi-process reduction hook of the optional tensor-parallel mode: an NCCL all-reduce over NVLink /
// NVSwitch, in place, on the plan's stream.  Kept out of libguffin_b200.so (which links only the CUDA
// runtime): this helper is loaded only where several processes shard one stream's model.
//
// gf_tp_unique_id   rank 0 makes the 128-byte id; the host hands it to the other ranks (any channel)
// gf_tp_create      every rank joins with the device it has made current
// gf_tp_reduce      a gf_reduce_fn: `user` is the communicator; sums `count` floats across the ranks in place
#include <cuda_runtime.h>
#include <nccl.h>

#include <cstdint>
#include <cstring>

static_assert(sizeof(ncclUniqueId) == 128, "the id travels as 128 bytes");

extern "C" {

__attribute__((visibility("default"))) int gf_tp_unique_id(void* out_id) {
    if (!out_id) return -1;
    ncclUniqueId id;
    if (ncclGetUniqueId(&id) != ncclSuccess) return -3;
    std::memcpy(out_id, &id, sizeof id);
    return 0;
}

__attribute__((visibility("default"))) int gf_tp_create(const void* id_bytes, int rank, int size, void** out_comm) {
    if (!id_bytes || !out_comm || size < 1 || rank < 0 || rank >= size) return -1;
    ncclUniqueId id;
    std::memcpy(&id, id_bytes, sizeof id);
    ncclComm_t comm = nullptr;
    if (ncclCommInitRank(&comm, size, id, rank) != ncclSuccess) return -3;
    *out_comm = comm;
    return 0;
}

__attribute__((visibility("default"))) int gf_tp_reduce(void* user, float* buffer_dev, uint64_t count, void* stream) {
    if (!user || !buffer_dev) return -1;
    return ncclAllReduce(buffer_dev, buffer_dev, (size_t)count, ncclFloat, ncclSum, static_cast<ncclComm_t>(user),
                         static_cast<cudaStream_t>(stream)) == ncclSuccess ? 0 : -3;
}

__attribute__((visibility("default"))) int gf_tp_destroy(void* comm) {
    if (comm) ncclCommDestroy(static_cast<ncclComm_t>(comm));
    return 0;
}

}  // extern "C"
