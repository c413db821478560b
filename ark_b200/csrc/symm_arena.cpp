// Symmetric, multicast-bound arena (see symm_arena.hpp). Driver entry points are looked up at run time, so the
// library still loads on hosts without a driver.
#include "symm_arena.hpp"

#include <cuda.h>
#include <cuda_runtime.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <vector>

#include "plan.hpp"

namespace arkb {

namespace {

template <typename F>
F driver_fn(const char *name) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
    return reinterpret_cast<F>(p);
}

struct Driver {
    CUresult (*DeviceGet)(CUdevice *, int);
    CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice);
    CUresult (*MemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
    CUresult (*MemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
    CUresult (*MemExportToShareableHandle)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType);
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *);
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*MulticastGetGranularity)(size_t *, const CUmulticastObjectProp *, CUmulticastGranularity_flags);
    bool ok = false;
};

const Driver &driver() {
    static Driver d = [] {
        Driver x;
        std::memset(&x, 0, sizeof(x));
#define ARKB_DRV(field, name) x.field = driver_fn<decltype(x.field)>(name)
        ARKB_DRV(DeviceGet, "cuDeviceGet");
        ARKB_DRV(DeviceGetAttribute, "cuDeviceGetAttribute");
        ARKB_DRV(MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
        ARKB_DRV(MemCreate, "cuMemCreate");
        ARKB_DRV(MemRelease, "cuMemRelease");
        ARKB_DRV(MemAddressReserve, "cuMemAddressReserve");
        ARKB_DRV(MemAddressFree, "cuMemAddressFree");
        ARKB_DRV(MemMap, "cuMemMap");
        ARKB_DRV(MemUnmap, "cuMemUnmap");
        ARKB_DRV(MemSetAccess, "cuMemSetAccess");
        ARKB_DRV(MemExportToShareableHandle, "cuMemExportToShareableHandle");
        ARKB_DRV(MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
        ARKB_DRV(MulticastCreate, "cuMulticastCreate");
        ARKB_DRV(MulticastAddDevice, "cuMulticastAddDevice");
        ARKB_DRV(MulticastBindMem, "cuMulticastBindMem");
        ARKB_DRV(MulticastUnbind, "cuMulticastUnbind");
        ARKB_DRV(MulticastGetGranularity, "cuMulticastGetGranularity");
#undef ARKB_DRV
        x.ok = x.DeviceGet && x.DeviceGetAttribute && x.MemGetAllocationGranularity && x.MemCreate && x.MemRelease &&
               x.MemAddressReserve && x.MemAddressFree && x.MemMap && x.MemUnmap && x.MemSetAccess &&
               x.MemExportToShareableHandle && x.MemImportFromShareableHandle && x.MulticastCreate && x.MulticastAddDevice &&
               x.MulticastBindMem && x.MulticastUnbind && x.MulticastGetGranularity;
        return x;
    }();
    return d;
}

void check(CUresult r, const char *what) {
    if (r != CUDA_SUCCESS) throw Error(E_GPU, std::string(what) + " failed with driver code " + std::to_string((int)r));
}

// ---- file descriptors between the rank processes: unix sockets in the abstract namespace -------------
struct SockName {
    char name[64];  // without the leading NUL of the abstract namespace
};

int make_listener(SockName &out) {
    static std::atomic<int> counter{0};
    std::memset(&out, 0, sizeof(out));
    snprintf(out.name, sizeof(out.name), "arkb.%d.%d", (int)getpid(), counter.fetch_add(1));
    const int s = socket(AF_UNIX, SOCK_STREAM, 0);
    if (s < 0) throw Error(E_SYSTEM, "socket() failed");
    sockaddr_un addr;
    std::memset(&addr, 0, sizeof(addr));
    addr.sun_family = AF_UNIX;
    std::strncpy(addr.sun_path + 1, out.name, sizeof(addr.sun_path) - 2);
    const socklen_t len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + std::strlen(out.name));
    if (bind(s, reinterpret_cast<sockaddr *>(&addr), len) != 0 || listen(s, 64) != 0) {
        close(s);
        throw Error(E_SYSTEM, "cannot listen on a unix socket for handle exchange");
    }
    return s;
}

void send_fd(const SockName &to, int fd, int tag) {
    const int s = socket(AF_UNIX, SOCK_STREAM, 0);
    if (s < 0) throw Error(E_SYSTEM, "socket() failed");
    sockaddr_un addr;
    std::memset(&addr, 0, sizeof(addr));
    addr.sun_family = AF_UNIX;
    std::strncpy(addr.sun_path + 1, to.name, sizeof(addr.sun_path) - 2);
    const socklen_t len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + std::strlen(to.name));
    if (connect(s, reinterpret_cast<sockaddr *>(&addr), len) != 0) {
        close(s);
        throw Error(E_SYSTEM, "cannot reach a peer's unix socket for handle exchange");
    }
    msghdr msg;
    std::memset(&msg, 0, sizeof(msg));
    iovec iov{&tag, sizeof(tag)};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr *c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
    const ssize_t n = sendmsg(s, &msg, 0);
    close(s);
    if (n != (ssize_t)sizeof(tag)) throw Error(E_SYSTEM, "sending a memory handle to a peer failed");
}

int recv_fd(int listener, int &tag) {
    const int s = accept(listener, nullptr, nullptr);
    if (s < 0) throw Error(E_SYSTEM, "accept() failed during handle exchange");
    msghdr msg;
    std::memset(&msg, 0, sizeof(msg));
    iovec iov{&tag, sizeof(tag)};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    const ssize_t n = recvmsg(s, &msg, 0);
    close(s);
    cmsghdr *c = CMSG_FIRSTHDR(&msg);
    if (n != (ssize_t)sizeof(tag) || !c || c->cmsg_type != SCM_RIGHTS) throw Error(E_SYSTEM, "receiving a memory handle from a peer failed");
    int fd = -1;
    std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
    return fd;
}

// Every rank learns whether all ranks are fine; throws the same error everywhere otherwise.
void agree(bool ok, const SymmArena::Allgather &ag, int world, const std::string &what) {
    int mine = ok ? 1 : 0;
    std::vector<int> all(world, 0);
    if (ag(&mine, all.data(), sizeof(int)) != 0) throw Error(E_SYSTEM, "bootstrap allgather failed");
    for (int v : all)
        if (!v) throw Error(E_UNSUPPORTED, what);
}

}  // namespace

bool SymmArena::device_supports(int device_id) {
    const Driver &d = driver();
    if (!d.ok) return false;
    CUdevice dev;
    int v = 0;
    if (d.DeviceGet(&dev, device_id) != CUDA_SUCCESS) return false;
    if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS || !v) return false;
    if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) != CUDA_SUCCESS || !v) return false;
    return true;
}

SymmArena::~SymmArena() {
    // without a rendezvous: last resort when the owner forgot destroy()
    if (active_) {
        try {
            destroy(nullptr);
        } catch (...) {
        }
    }
}

void SymmArena::create(int device_id, int rank, int world, size_t bytes, const Allgather &ag) {
    const Driver &d = driver();
    device_ = device_id;
    rank_ = rank;
    world_ = world;
    agree(device_supports(device_id), ag, world, "a rank's device or driver cannot take part in an NVSwitch multicast object");
    CUdevice dev;
    check(d.DeviceGet(&dev, device_id), "cuDeviceGet");
    CUmemAllocationProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device_id;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmulticastObjectProp mprop;
    std::memset(&mprop, 0, sizeof(mprop));
    mprop.numDevices = (unsigned)world;
    mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t g_mem = 0, g_mc = 0;
    check(d.MemGetAllocationGranularity(&g_mem, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    mprop.size = std::max<size_t>(bytes, 1);
    check(d.MulticastGetGranularity(&g_mc, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
    const size_t gran = std::max(g_mem, g_mc);
    // the same size on every rank: the largest request, rounded to the granularity
    uint64_t mine = (std::max<size_t>(bytes, 1) + gran - 1) / gran * gran;
    std::vector<uint64_t> sizes(world);
    if (ag(&mine, sizes.data(), sizeof(uint64_t)) != 0) throw Error(E_SYSTEM, "bootstrap allgather failed");
    for (auto v : sizes) mine = std::max(mine, v);
    bytes_ = (size_t)mine;
    mprop.size = bytes_;

    CUmemAccessDesc access;
    std::memset(&access, 0, sizeof(access));
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device_id;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    auto map = [&](CUmemGenericAllocationHandle h) -> char * {
        CUdeviceptr va = 0;
        check(d.MemAddressReserve(&va, bytes_, gran, 0, 0), "cuMemAddressReserve");
        CUresult r = d.MemMap(va, bytes_, 0, h, 0);
        if (r == CUDA_SUCCESS) r = d.MemSetAccess(va, bytes_, &access, 1);
        if (r != CUDA_SUCCESS) {
            d.MemAddressFree(va, bytes_);
            check(r, "cuMemMap / cuMemSetAccess");
        }
        return reinterpret_cast<char *>(va);
    };

    int listener = -1, my_fd = -1, mc_fd = -1;
    std::string err;
    try {
        CUmemGenericAllocationHandle h = 0;
        check(d.MemCreate(&h, bytes_, &prop, 0), "cuMemCreate");
        h_local_ = h;
        local_ = map(h);
        if (cudaMemset(local_, 0, bytes_) != cudaSuccess) throw Error(E_GPU, "cudaMemset of the arena failed");
        peer_[rank] = local_;
        // exchange: socket names, then one descriptor to every peer
        SockName me;
        listener = make_listener(me);
        std::vector<SockName> names(world);
        if (ag(&me, names.data(), sizeof(SockName)) != 0) throw Error(E_SYSTEM, "bootstrap allgather failed");
        check(d.MemExportToShareableHandle(&my_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
        for (int r = 0; r < world; ++r)
            if (r != rank) send_fd(names[r], my_fd, r == rank ? -1 : rank);
        if (rank == 0) {
            CUmemGenericAllocationHandle mc = 0;
            check(d.MulticastCreate(&mc, &mprop), "cuMulticastCreate");
            h_mc_ = mc;
            check(d.MemExportToShareableHandle(&mc_fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle (multicast)");
            for (int r = 1; r < world; ++r) send_fd(names[r], mc_fd, 1000);
        }
        const int expect = (world - 1) + (rank == 0 ? 0 : 1);
        for (int i = 0; i < expect; ++i) {
            int tag = -1;
            const int fd = recv_fd(listener, tag);
            CUmemGenericAllocationHandle ih = 0;
            const CUresult r = d.MemImportFromShareableHandle(&ih, reinterpret_cast<void *>((uintptr_t)fd), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            close(fd);
            check(r, "cuMemImportFromShareableHandle");
            if (tag == 1000) {
                h_mc_ = ih;
            } else if (tag >= 0 && tag < world && tag != rank) {
                h_peer_[tag] = ih;
                peer_[tag] = map(ih);
            } else {
                throw Error(E_SYSTEM, "unexpected message during handle exchange");
            }
        }
        check(d.MulticastAddDevice(h_mc_, dev), "cuMulticastAddDevice");
    } catch (const Error &e) {
        err = e.what();
    }
    if (listener >= 0) close(listener);
    if (my_fd >= 0) close(my_fd);
    if (mc_fd >= 0) close(mc_fd);
    active_ = true;  // so that destroy() below releases what exists
    try {
        agree(err.empty(), ag, world, "setting up the symmetric arena failed on a rank" + (err.empty() ? std::string() : ": " + err));
        // every device has been added: bind, then (after every rank has bound) map the multicast address
        CUresult r = d.MulticastBindMem(h_mc_, 0, h_local_, 0, bytes_, 0);
        bound_ = r == CUDA_SUCCESS;
        agree(bound_, ag, world, "cuMulticastBindMem failed on a rank (code " + std::to_string((int)r) + ")");
        mc_ = map(h_mc_);
        agree(true, ag, world, "");
    } catch (...) {
        destroy(nullptr);
        throw;
    }
}

void SymmArena::destroy(const Allgather &ag) {
    if (!active_) return;
    const Driver &d = driver();
    // no rank may unbind while another rank's kernel could still use the multicast address
    if (ag) {
        int mine = rank_;
        std::vector<int> all(world_);
        ag(&mine, all.data(), sizeof(int));
    }
    cudaDeviceSynchronize();
    CUdevice dev;
    if (mc_) {
        d.MemUnmap(reinterpret_cast<CUdeviceptr>(mc_), bytes_);
        d.MemAddressFree(reinterpret_cast<CUdeviceptr>(mc_), bytes_);
        mc_ = nullptr;
    }
    if (bound_ && d.DeviceGet(&dev, device_) == CUDA_SUCCESS) d.MulticastUnbind(h_mc_, dev, 0, bytes_);
    bound_ = false;
    if (h_mc_) d.MemRelease(h_mc_);
    h_mc_ = 0;
    for (int r = 0; r < kMaxPeers; ++r) {
        if (r != rank_ && peer_[r]) {
            d.MemUnmap(reinterpret_cast<CUdeviceptr>(peer_[r]), bytes_);
            d.MemAddressFree(reinterpret_cast<CUdeviceptr>(peer_[r]), bytes_);
            if (h_peer_[r]) d.MemRelease(h_peer_[r]);
        }
        peer_[r] = nullptr;
        h_peer_[r] = 0;
    }
    if (local_) {
        d.MemUnmap(reinterpret_cast<CUdeviceptr>(local_), bytes_);
        d.MemAddressFree(reinterpret_cast<CUdeviceptr>(local_), bytes_);
        local_ = nullptr;
    }
    if (h_local_) d.MemRelease(h_local_);
    h_local_ = 0;
    active_ = false;
}

}  // namespace arkb
