// Collectives of the reference's distributed API (include/tensorcore/distributed.h:51-87) on
// device buffers, over NCCL.  The reference ships a TCP ring between hosts
// (lib/distributed/distributed_cpu.cpp:202-347); on one NVSwitch box the same calls map onto
// ncclAllReduce / ncclBroadcast / ncclAllGather between one process per GPU.
//
// NCCL is not linked: libnccl.so.2 is opened on the first tc_dist_init with more than one rank,
// so a process that never uses the collectives needs no NCCL at all.  The ranks find each other
// through the rendezvous URL ("...://host:port"): rank 0 listens there and hands NCCL's 128-byte
// unique id to every other rank over TCP; nothing else crosses that socket.
#include "kernels.h"

#include <arpa/inet.h>
#include <dlfcn.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <thread>

namespace tcb {
namespace {

constexpr int kIdBytes = 128;
struct UniqueId { char internal[kIdBytes]; };
typedef struct ncclComm* Comm;

struct Nccl {
    void* lib = nullptr;
    int (*GetUniqueId)(UniqueId*) = nullptr;
    int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(Comm) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, Comm, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

Nccl* load_nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {std::getenv("TC_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char* name : names) {
            if (!name || !name[0]) continue;
            n.lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (n.lib) break;
        }
        if (!n.lib) return;
#define TCB_SYM(field, sym) n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.lib, sym))
        TCB_SYM(GetUniqueId, "ncclGetUniqueId");
        TCB_SYM(CommInitRank, "ncclCommInitRank");
        TCB_SYM(CommDestroy, "ncclCommDestroy");
        TCB_SYM(AllReduce, "ncclAllReduce");
        TCB_SYM(Broadcast, "ncclBroadcast");
        TCB_SYM(AllGather, "ncclAllGather");
        TCB_SYM(GetErrorString, "ncclGetErrorString");
#undef TCB_SYM
        if (!n.GetUniqueId || !n.CommInitRank || !n.CommDestroy || !n.AllReduce || !n.Broadcast || !n.AllGather) {
            dlclose(n.lib);
            n.lib = nullptr;
        }
    });
    return n.lib ? &n : nullptr;
}

// "scheme://host:port[/anything]" or "host:port"
bool parse_url(const char* url, std::string* host, int* port) {
    if (!url) return false;
    std::string s(url);
    const size_t sch = s.find("://");
    if (sch != std::string::npos) s = s.substr(sch + 3);
    const size_t slash = s.find('/');
    if (slash != std::string::npos) s = s.substr(0, slash);
    const size_t colon = s.rfind(':');
    if (colon == std::string::npos || colon == 0 || colon + 1 >= s.size()) return false;
    *host = s.substr(0, colon);
    *port = std::atoi(s.c_str() + colon + 1);
    return *port > 0 && *port < 65536;
}

bool send_all(int fd, const void* p, size_t n) {
    const char* c = static_cast<const char*>(p);
    while (n) {
        const ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
        if (k <= 0) return false;
        c += k; n -= static_cast<size_t>(k);
    }
    return true;
}
bool recv_all(int fd, void* p, size_t n) {
    char* c = static_cast<char*>(p);
    while (n) {
        const ssize_t k = ::recv(fd, c, n, 0);
        if (k <= 0) return false;
        c += k; n -= static_cast<size_t>(k);
    }
    return true;
}

// Rank 0 serves the id to world - 1 connections; the others fetch it (retrying while rank 0 is not
// listening yet).  Both sides give up after `timeout_s`.
bool exchange_id(UniqueId* id, int world, int rank, const std::string& host, int port, int timeout_s) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(timeout_s);
    if (rank == 0) {
        const int ls = ::socket(AF_INET, SOCK_STREAM, 0);
        if (ls < 0) return false;
        int one = 1;
        setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        sockaddr_in addr{};
        addr.sin_family = AF_INET;
        addr.sin_addr.s_addr = htonl(INADDR_ANY);
        addr.sin_port = htons(static_cast<uint16_t>(port));
        if (::bind(ls, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(ls, world) != 0) {
            ::close(ls);
            return false;
        }
        timeval tv{1, 0};
        setsockopt(ls, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        int served = 0;
        while (served < world - 1 && std::chrono::steady_clock::now() < deadline) {
            const int fd = ::accept(ls, nullptr, nullptr);
            if (fd < 0) continue;
            int peer = -1;
            const bool ok = recv_all(fd, &peer, sizeof(peer)) && send_all(fd, id, sizeof(*id));
            ::close(fd);
            if (ok) ++served;
        }
        ::close(ls);
        return served == world - 1;
    }
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || !res) return false;
    bool done = false;
    while (!done && std::chrono::steady_clock::now() < deadline) {
        const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
        if (fd < 0) break;
        if (::connect(fd, res->ai_addr, res->ai_addrlen) == 0)
            done = send_all(fd, &rank, sizeof(rank)) && recv_all(fd, id, sizeof(*id));
        ::close(fd);
        if (!done) std::this_thread::sleep_for(std::chrono::milliseconds(100));
    }
    freeaddrinfo(res);
    return done;
}

}  // namespace

struct DistComm {
    int world = 1, rank = 0;
    Comm comm = nullptr;
    Nccl* nccl = nullptr;
    float* scratch = nullptr;   // one float on the device: what the barrier reduces
};

// 0 on success; -1 bad arguments, -2 NCCL unavailable, -3 rendezvous failed, -4 NCCL error.
int dist_create(int world, int rank, const char* url, DistComm** out) {
    if (!out || world < 1 || rank < 0 || rank >= world) return -1;
    DistComm* d = new (std::nothrow) DistComm();
    if (!d) return -4;
    d->world = world;
    d->rank = rank;
    if (world == 1) { *out = d; return 0; }
    std::string host;
    int port = 0;
    if (!parse_url(url, &host, &port)) { delete d; return -1; }
    d->nccl = load_nccl();
    if (!d->nccl) { delete d; return -2; }
    UniqueId id;
    std::memset(&id, 0, sizeof(id));
    if (rank == 0 && d->nccl->GetUniqueId(&id) != 0) { delete d; return -4; }
    const char* t = std::getenv("TC_DIST_TIMEOUT_S");
    if (!exchange_id(&id, world, rank, host, port, t ? std::atoi(t) : 120)) { delete d; return -3; }
    if (d->nccl->CommInitRank(&d->comm, world, id, rank) != 0) { delete d; return -4; }
    if (cudaMalloc(reinterpret_cast<void**>(&d->scratch), sizeof(float)) != cudaSuccess ||
        cudaMemset(d->scratch, 0, sizeof(float)) != cudaSuccess) {
        d->nccl->CommDestroy(d->comm);
        delete d;
        return -4;
    }
    *out = d;
    return 0;
}

void dist_destroy(DistComm* d) {
    if (!d) return;
    if (d->comm) d->nccl->CommDestroy(d->comm);
    if (d->scratch) cudaFree(d->scratch);
    delete d;
}

int dist_world(const DistComm* d) { return d ? d->world : 0; }
int dist_rank(const DistComm* d) { return d ? d->rank : -1; }

// dtype: 0 = fp16, 2 = fp32 (tc_dtype_t values); op: 0 sum, 1 avg, 2 max, 3 min (tc_reduce_op_t).
static int nccl_type(int dtype) { return dtype == 0 ? 6 : (dtype == 2 ? 7 : -1); }
static int nccl_op(int op) { return op == 0 ? 0 : (op == 1 ? 4 : (op == 2 ? 2 : (op == 3 ? 3 : -1))); }

int dist_allreduce(DistComm* d, void* buf, size_t count, int dtype, int op, cudaStream_t st) {
    if (!d || !buf || nccl_type(dtype) < 0 || nccl_op(op) < 0) return -1;
    if (d->world == 1) return 0;
    return d->nccl->AllReduce(buf, buf, count, nccl_type(dtype), nccl_op(op), d->comm, st) == 0 ? 0 : -4;
}
int dist_broadcast(DistComm* d, void* buf, size_t count, int dtype, int root, cudaStream_t st) {
    if (!d || !buf || nccl_type(dtype) < 0 || root < 0 || root >= d->world) return -1;
    if (d->world == 1) return 0;
    return d->nccl->Broadcast(buf, buf, count, nccl_type(dtype), root, d->comm, st) == 0 ? 0 : -4;
}
int dist_allgather(DistComm* d, const void* in, void* out, size_t count_per_rank, int dtype, cudaStream_t st) {
    if (!d || !in || !out || nccl_type(dtype) < 0) return -1;
    if (d->world == 1) {
        const size_t bytes = count_per_rank * (dtype == 0 ? 2 : 4);
        return cudaMemcpyAsync(out, in, bytes, cudaMemcpyDeviceToDevice, st) == cudaSuccess ? 0 : -4;
    }
    return d->nccl->AllGather(in, out, count_per_rank, nccl_type(dtype), d->comm, st) == 0 ? 0 : -4;
}
int dist_barrier(DistComm* d, cudaStream_t st) {
    if (!d) return -1;
    if (d->world == 1) return 0;
    return d->nccl->AllReduce(d->scratch, d->scratch, 1, 7, 0, d->comm, st) == 0 ? 0 : -4;
}

}  // namespace tcb
