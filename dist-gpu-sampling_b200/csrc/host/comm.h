// Bootstrap communicator shared by the store code (host only).
#pragma once
#include <cstddef>

namespace dgs {
// Both are collective, synchronous and only used while a ChunkTensor is
// created or destroyed; with no communicator set they are single-rank no-ops.
int comm_broadcast_bytes(void* buf, size_t nbytes, int root);
int comm_allgather_bytes(const void* send, void* recv, size_t nbytes_per_rank);
}  // namespace dgs
