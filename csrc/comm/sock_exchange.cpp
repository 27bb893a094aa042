#include "sock_exchange.h"

#include <arpa/inet.h>
#include <cerrno>
#include <cstring>
#include <fstream>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <set>
#include <sys/socket.h>
#include <unistd.h>

#include "tilexr_log.h"
#include "tilexr_types.h"

namespace TileXR {

namespace {

bool SendAll(int fd, const void *buf, size_t bytes)
{
    const char *p = static_cast<const char *>(buf);
    while (bytes > 0) {
        ssize_t n = ::send(fd, p, bytes, MSG_NOSIGNAL);
        if (n < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += n;
        bytes -= static_cast<size_t>(n);
    }
    return true;
}

bool RecvAll(int fd, void *buf, size_t bytes)
{
    char *p = static_cast<char *>(buf);
    while (bytes > 0) {
        ssize_t n = ::recv(fd, p, bytes, 0);
        if (n == 0) return false;
        if (n < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += n;
        bytes -= static_cast<size_t>(n);
    }
    return true;
}

constexpr uint64_t HELLO_MAGIC = 0x5458524c4f434b31ull;   // handshake word

} // namespace

int Exchange::Barrier()
{
    char token = 1;
    std::vector<char> all(4096);
    // rank count is unknown here; AllGather implementations size by their own rankSize, and a
    // 4 KiB buffer covers the 128-rank limit.
    return AllGather(&token, all.data(), 1);
}

SockExchange::SockExchange(int rank, int rankSize, const std::string &ip, uint16_t port)
    : rank_(rank), rankSize_(rankSize), ip_(ip), port_(port)
{
}

SockExchange::~SockExchange()
{
    for (int fd : peers_) {
        if (fd >= 0) ::close(fd);
    }
    if (listenFd_ >= 0) ::close(listenFd_);
}

bool SockExchange::ParseCommId(const char *text, std::string *ip, uint16_t *port)
{
    *ip = "127.0.0.1";
    *port = 10067;
    if (text == nullptr || *text == '\0') return true;
    std::string s(text);
    const size_t colon = s.rfind(':');
    if (colon == std::string::npos) return false;
    const std::string host = s.substr(0, colon);
    const std::string portText = s.substr(colon + 1);
    if (host.empty() || portText.empty()) return false;
    char *end = nullptr;
    const long p = std::strtol(portText.c_str(), &end, 10);
    if (*end != '\0' || p <= 0 || p > 65535) return false;
    in_addr addr;
    if (inet_pton(AF_INET, host.c_str(), &addr) != 1) return false;
    *ip = host;
    *port = static_cast<uint16_t>(p);
    return true;
}

std::string SockExchange::ReadBootId()
{
    std::ifstream f("/proc/sys/kernel/random/boot_id");
    std::string id;
    if (f) std::getline(f, id);
    if (id.empty()) id = "unknown-boot-id";
    return id;
}

int SockExchange::Prepare()
{
    if (ready_) return TILEXR_SUCCESS;
    if (rankSize_ <= 1) {
        ready_ = true;
        return TILEXR_SUCCESS;
    }
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(port_);
    if (inet_pton(AF_INET, ip_.c_str(), &addr.sin_addr) != 1) {
        TILEXR_LOG(ERROR) << "bad bootstrap address " << ip_;
        return TILEXR_ERROR_PARA_CHECK_FAIL;
    }
    const int one = 1;
    if (rank_ == 0) {
        listenFd_ = ::socket(AF_INET, SOCK_STREAM, 0);
        if (listenFd_ < 0) return TILEXR_ERROR_INTERNAL;
        ::setsockopt(listenFd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        if (::bind(listenFd_, reinterpret_cast<sockaddr *>(&addr), sizeof(addr)) != 0 ||
            ::listen(listenFd_, rankSize_) != 0) {
            TILEXR_LOG(ERROR) << "rank 0 cannot listen on " << ip_ << ":" << port_ << ": " << std::strerror(errno);
            return TILEXR_ERROR_INTERNAL;
        }
        peers_.assign(rankSize_, -1);
        timeval tv{connectRetries, 0};
        ::setsockopt(listenFd_, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        for (int i = 1; i < rankSize_; ++i) {
            int fd = ::accept(listenFd_, nullptr, nullptr);
            if (fd < 0) {
                TILEXR_LOG(ERROR) << "accept failed after " << (i - 1) << " clients: " << std::strerror(errno);
                return TILEXR_ERROR_TIMEOUT;
            }
            ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            uint64_t hello[2] = {0, 0};
            if (!RecvAll(fd, hello, sizeof(hello)) || hello[0] != HELLO_MAGIC || hello[1] == 0 ||
                hello[1] >= static_cast<uint64_t>(rankSize_) || peers_[hello[1]] != -1) {
                TILEXR_LOG(ERROR) << "bad handshake from a bootstrap client";
                ::close(fd);
                return TILEXR_ERROR_INTERNAL;
            }
            peers_[hello[1]] = fd;
        }
    } else {
        int fd = -1;
        for (int attempt = 0; attempt < connectRetries; ++attempt) {
            fd = ::socket(AF_INET, SOCK_STREAM, 0);
            if (fd < 0) return TILEXR_ERROR_INTERNAL;
            if (::connect(fd, reinterpret_cast<sockaddr *>(&addr), sizeof(addr)) == 0) break;
            ::close(fd);
            fd = -1;
            ::usleep(attempt < 50 ? 20 * 1000 : 1000 * 1000);
        }
        if (fd < 0) {
            TILEXR_LOG(ERROR) << "rank " << rank_ << " cannot reach rank 0 at " << ip_ << ":" << port_;
            return TILEXR_ERROR_TIMEOUT;
        }
        ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        const uint64_t hello[2] = {HELLO_MAGIC, static_cast<uint64_t>(rank_)};
        if (!SendAll(fd, hello, sizeof(hello))) {
            ::close(fd);
            return TILEXR_ERROR_INTERNAL;
        }
        peers_.assign(1, fd);
    }
    ready_ = true;
    return TILEXR_SUCCESS;
}

int SockExchange::AllGather(const void *send, void *recv, size_t bytes)
{
    int ret = Prepare();
    if (ret != TILEXR_SUCCESS) return ret;
    char *out = static_cast<char *>(recv);
    if (rankSize_ <= 1) {
        std::memcpy(out, send, bytes);
        return TILEXR_SUCCESS;
    }
    if (rank_ == 0) {
        std::memcpy(out, send, bytes);
        for (int r = 1; r < rankSize_; ++r) {
            if (!RecvAll(peers_[r], out + static_cast<size_t>(r) * bytes, bytes)) {
                TILEXR_LOG(ERROR) << "bootstrap: lost rank " << r << " during gather";
                return TILEXR_ERROR_INTERNAL;
            }
        }
        for (int r = 1; r < rankSize_; ++r) {
            if (!SendAll(peers_[r], out, bytes * rankSize_)) return TILEXR_ERROR_INTERNAL;
        }
    } else {
        if (!SendAll(peers_[0], send, bytes) || !RecvAll(peers_[0], out, bytes * rankSize_)) {
            TILEXR_LOG(ERROR) << "bootstrap: rank " << rank_ << " lost rank 0";
            return TILEXR_ERROR_INTERNAL;
        }
    }
    return TILEXR_SUCCESS;
}

int SockExchange::GetNodeNum(int *nodeNum)
{
    char mine[64] = {};
    const std::string id = ReadBootId();
    std::strncpy(mine, id.c_str(), sizeof(mine) - 1);
    std::vector<char> all(static_cast<size_t>(rankSize_) * sizeof(mine));
    int ret = AllGather(mine, all.data(), sizeof(mine));
    if (ret != TILEXR_SUCCESS) return ret;
    std::set<std::string> distinct;
    for (int r = 0; r < rankSize_; ++r) distinct.insert(std::string(all.data() + r * sizeof(mine)));
    *nodeNum = static_cast<int>(distinct.size());
    return TILEXR_SUCCESS;
}

} // namespace TileXR
