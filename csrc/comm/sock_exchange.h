// Bootstrap exchange over TCP: rank 0 listens, the other ranks connect, and AllGather is a
// star (gather to rank 0, scatter the concatenation back).  Used once at communicator
// bring-up to trade device ids, process ids and memory handles, so simplicity beats speed.
// Behaviour follows the reference (src/comm/tools/socket/tilexr_sock_exchange.h:38-197):
// address from TILEXR_COMM_ID ("ip:port", default 127.0.0.1:10067) plus the communicator
// domain as a port offset, clients retry the connect for 180 s, node count = number of
// distinct kernel boot ids.
#ifndef TILEXR_SOCK_EXCHANGE_H
#define TILEXR_SOCK_EXCHANGE_H

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace TileXR {

// Abstract all-gather used by communicator bring-up; implemented over TCP here and over a
// torch Store in the Python binding.
class Exchange {
public:
    virtual ~Exchange() = default;
    // Every rank contributes `bytes` bytes; `recv` receives rankSize*bytes in rank order.
    virtual int AllGather(const void *send, void *recv, size_t bytes) = 0;
    int Barrier();
};

class SockExchange : public Exchange {
public:
    SockExchange(int rank, int rankSize, const std::string &ip, uint16_t port);
    ~SockExchange() override;

    int Prepare();                                   // listen/accept or connect; idempotent
    int AllGather(const void *send, void *recv, size_t bytes) override;
    int GetNodeNum(int *nodeNum);                    // distinct boot ids among the ranks

    static bool ParseCommId(const char *text, std::string *ip, uint16_t *port);
    static std::string ReadBootId();

    int connectRetries = 180;                        // one second apart
private:
    int rank_;
    int rankSize_;
    std::string ip_;
    uint16_t port_;
    int listenFd_ = -1;
    std::vector<int> peers_;   // rank 0: fd per client rank; others: peers_[0] = fd to rank 0
    bool ready_ = false;
};

// Exchange backed by a caller-supplied function (TCPStore, process group, MPI...).
typedef int (*AllGatherCallback)(void *ctx, const void *send, void *recv, size_t bytesPerRank);
class CallbackExchange : public Exchange {
public:
    CallbackExchange(AllGatherCallback fn, void *ctx) : fn_(fn), ctx_(ctx) {}
    int AllGather(const void *send, void *recv, size_t bytes) override { return fn_(ctx_, send, recv, bytes); }
private:
    AllGatherCallback fn_;
    void *ctx_;
};

} // namespace TileXR

#endif
