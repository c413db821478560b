// A rank's arena as a symmetric, multicast-capable allocation (NVLink SHARP / NVLS).
//
// The default arena is one cudaMalloc per rank, mapped into the peers with CUDA IPC handles; that serves plain peer
// loads and stores. In-switch reductions (multimem.ld_reduce) and one-store broadcasts (multimem.st) need more: every
// rank's memory must be bound, at the same offset, to one NVSwitch multicast object, and only memory created with the
// virtual-memory-management API can be bound. SymmArena allocates the arena that way, hands it to the peers as a
// POSIX file descriptor (sent over a unix socket: such allocations have no CUDA IPC handle), builds the multicast
// object over all ranks and maps it. It is used only when the executor is asked for NVLS (ARKB_NVLS=1) and the
// device and every rank support it; otherwise the executor keeps the cudaMalloc arena.
#pragma once
#include <cstddef>
#include <functional>
#include <string>

#include "program.h"

namespace arkb {

class SymmArena {
   public:
    using Allgather = std::function<int(const void *send, void *recv, size_t bytes)>;
    SymmArena() = default;
    ~SymmArena();
    SymmArena(const SymmArena &) = delete;
    SymmArena &operator=(const SymmArena &) = delete;

    // True when this device can take part in a multicast object (driver entry points present, attribute set).
    static bool device_supports(int device_id);

    // Collective over all ranks: allocates `bytes` (zero-filled) on `device_id`, maps every peer's allocation, creates
    // and maps the multicast object. Throws arkb::Error; on failure nothing stays allocated.
    void create(int device_id, int rank, int world, size_t bytes, const Allgather &allgather);
    // Collective: unbinds from the multicast object (after a rendezvous, so that no rank's kernel still uses it),
    // unmaps and releases everything. Safe to call twice.
    void destroy(const Allgather &allgather);

    bool active() const { return active_; }
    char *local() const { return local_; }
    char *peer(int r) const { return peer_[r]; }
    char *multicast() const { return mc_; }  // the multicast address of offset 0 of every rank's arena
    size_t bytes() const { return bytes_; }

   private:
    bool active_ = false;
    int device_ = 0, rank_ = 0, world_ = 1;
    size_t bytes_ = 0;
    char *local_ = nullptr, *mc_ = nullptr;
    char *peer_[kMaxPeers] = {};
    unsigned long long h_local_ = 0, h_mc_ = 0;
    unsigned long long h_peer_[kMaxPeers] = {};
    bool bound_ = false;
};

}  // namespace arkb
