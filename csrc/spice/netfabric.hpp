// TCP mesh between the solver processes of one partitioned run.
//
// Every process binds a listening socket, publishes "host:port" as a file in a rendezvous directory, waits
// for the files of the others, connects to every lower-numbered process and accepts the higher-numbered
// ones. After that each pair shares one stream and all traffic is length-prefixed messages.
//
// `exchange` is the only communication primitive the runner needs: send one message to each listed peer and
// receive one from each, making progress on all sockets at once (poll, non-blocking), so that no ordering of
// sends and receives between processes can deadlock and no message size depends on socket buffer sizes.
// Every wait has a deadline; a peer that closed its end, or that stays silent past the deadline, ends the
// call with an error that names it, so that the survivors of a crashed run stop by themselves.
//
// The reference moves these messages over in-process channels and never starts more than one solver that
// talks (nangila-spice/nangila-node/src/comm.rs:1-300, fabric.rs); this file is what makes the partitions
// separate processes.
#pragma once
#include <arpa/inet.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <string>
#include <thread>
#include <vector>

namespace nspice {

class SocketMesh {
public:
    struct Stats { uint64_t messages_sent = 0, bytes_sent = 0, messages_received = 0, bytes_received = 0; };
    Stats stats;
    std::string error;  // what went wrong in the last failing call

    SocketMesh(uint32_t id, uint32_t total, std::string rendezvous_dir, std::string bind_host = "127.0.0.1")
        : id_(id), total_(total), dir_(std::move(rendezvous_dir)), host_(std::move(bind_host)), fds_(total, -1) {}
    SocketMesh(const SocketMesh&) = delete;
    ~SocketMesh() { close_all(); }

    uint32_t id() const { return id_; }
    uint32_t total() const { return total_; }

    // Builds the full mesh. False (with `error` set) when a peer does not show up within the deadline.
    bool connect_all(int timeout_ms) {
        const auto deadline = now_ms() + timeout_ms;
        int listener = ::socket(AF_INET, SOCK_STREAM, 0);
        if (listener < 0) return fail("socket: " + errno_text());
        int one = 1;
        ::setsockopt(listener, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
        sockaddr_in addr{};
        addr.sin_family = AF_INET;
        addr.sin_port = 0;
        if (::inet_pton(AF_INET, host_.c_str(), &addr.sin_addr) != 1) { ::close(listener); return fail("bind address '" + host_ + "' is not an IPv4 address"); }
        if (::bind(listener, reinterpret_cast<sockaddr*>(&addr), sizeof addr) != 0 || ::listen(listener, int(total_)) != 0) {
            std::string e = errno_text();
            ::close(listener);
            return fail("bind/listen on " + host_ + ": " + e);
        }
        socklen_t len = sizeof addr;
        ::getsockname(listener, reinterpret_cast<sockaddr*>(&addr), &len);
        const int port = ntohs(addr.sin_port);
        // publish: write to a temporary name, then rename, so that a reader never sees half a file
        {
            ::mkdir(dir_.c_str(), 0777);
            const std::string tmp = dir_ + "/.node_" + std::to_string(id_) + ".tmp", fin = address_file(id_);
            std::ofstream f(tmp);
            f << host_ << ":" << port << "\n";
            f.close();
            if (!f || ::rename(tmp.c_str(), fin.c_str()) != 0) { ::close(listener); return fail("cannot publish " + fin + ": " + errno_text()); }
        }
        bool ok = true;
        // connect to the lower-numbered processes
        for (uint32_t p = 0; ok && p < id_; ++p) {
            std::string host;
            int pport = 0;
            while (!read_address(p, host, pport)) {
                if (now_ms() > deadline) { ok = fail("process " + std::to_string(p) + " did not publish its address in " + dir_); break; }
                std::this_thread::sleep_for(std::chrono::milliseconds(10));
            }
            if (!ok) break;
            int fd = -1;
            while (true) {
                fd = ::socket(AF_INET, SOCK_STREAM, 0);
                sockaddr_in pa{};
                pa.sin_family = AF_INET;
                pa.sin_port = htons(uint16_t(pport));
                ::inet_pton(AF_INET, host.c_str(), &pa.sin_addr);
                if (::connect(fd, reinterpret_cast<sockaddr*>(&pa), sizeof pa) == 0) break;
                ::close(fd);
                fd = -1;
                if (now_ms() > deadline) { ok = fail("cannot connect to process " + std::to_string(p) + " at " + host + ":" + std::to_string(pport) + ": " + errno_text()); break; }
                std::this_thread::sleep_for(std::chrono::milliseconds(10));
            }
            if (!ok) break;
            uint32_t me = id_;
            if (::send(fd, &me, sizeof me, MSG_NOSIGNAL) != ssize_t(sizeof me)) { ::close(fd); ok = fail("handshake with process " + std::to_string(p) + ": " + errno_text()); break; }
            adopt(p, fd);
        }
        // accept the higher-numbered ones
        uint32_t expected = total_ - 1 - id_;
        while (ok && expected > 0) {
            pollfd pf{listener, POLLIN, 0};
            const long long left = deadline - now_ms();
            if (left <= 0 || ::poll(&pf, 1, int(std::min<long long>(left, 200))) < 0) {
                if (left <= 0) { ok = fail(std::to_string(expected) + " higher-numbered process(es) never connected"); break; }
                continue;
            }
            if (!(pf.revents & POLLIN)) continue;
            int fd = ::accept(listener, nullptr, nullptr);
            if (fd < 0) continue;
            uint32_t who = 0;
            timeval tv{2, 0};
            ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
            if (::recv(fd, &who, sizeof who, MSG_WAITALL) != ssize_t(sizeof who) || who <= id_ || who >= total_ || fds_[who] >= 0) { ::close(fd); continue; }
            adopt(who, fd);
            --expected;
        }
        ::close(listener);
        if (!ok) close_all();
        return ok;
    }

    // One message to every peer in `peers` (out[i] goes to peers[i]) and one from each (in[i] comes from peers[i]).
    bool exchange(const std::vector<uint32_t>& peers, const std::vector<std::string>& out, std::vector<std::string>& in, int timeout_ms) {
        struct Io { std::string tx; size_t sent = 0; char head[8]; size_t head_got = 0; uint64_t want = 0; size_t got = 0; bool rx_done = false; };
        std::vector<Io> io(peers.size());
        in.assign(peers.size(), std::string());
        for (size_t i = 0; i < peers.size(); ++i) {
            if (peers[i] >= total_ || peers[i] == id_ || fds_[peers[i]] < 0) return fail("no connection to process " + std::to_string(peers[i]));
            const uint64_t n = out[i].size();
            io[i].tx.assign(reinterpret_cast<const char*>(&n), 8);
            io[i].tx += out[i];
        }
        const auto deadline = now_ms() + timeout_ms;
        std::vector<pollfd> pfs(peers.size());
        while (true) {
            bool busy = false;
            for (size_t i = 0; i < peers.size(); ++i) {
                pfs[i].fd = fds_[peers[i]];
                pfs[i].events = 0;
                pfs[i].revents = 0;
                if (io[i].sent < io[i].tx.size()) pfs[i].events |= POLLOUT;
                if (!io[i].rx_done) pfs[i].events |= POLLIN;
                if (pfs[i].events) busy = true; else pfs[i].fd = -1;
            }
            if (!busy) break;
            const long long left = deadline - now_ms();
            if (left <= 0) {
                for (size_t i = 0; i < peers.size(); ++i)
                    if (!io[i].rx_done) return fail("no message from process " + std::to_string(peers[i]) + " within " + std::to_string(timeout_ms) + " ms");
                return fail("could not finish sending within " + std::to_string(timeout_ms) + " ms");
            }
            if (::poll(pfs.data(), nfds_t(pfs.size()), int(std::min<long long>(left, 500))) < 0) {
                if (errno == EINTR) continue;
                return fail("poll: " + errno_text());
            }
            for (size_t i = 0; i < peers.size(); ++i) {
                if (pfs[i].fd < 0) continue;
                Io& s = io[i];
                if ((pfs[i].revents & POLLOUT) && s.sent < s.tx.size()) {
                    ssize_t w = ::send(pfs[i].fd, s.tx.data() + s.sent, s.tx.size() - s.sent, MSG_NOSIGNAL | MSG_DONTWAIT);
                    if (w > 0) s.sent += size_t(w);
                    else if (w < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return fail("send to process " + std::to_string(peers[i]) + ": " + errno_text());
                }
                if ((pfs[i].revents & (POLLIN | POLLHUP | POLLERR)) && !s.rx_done) {
                    ssize_t r;
                    if (s.head_got < 8) {
                        r = ::recv(pfs[i].fd, s.head + s.head_got, 8 - s.head_got, MSG_DONTWAIT);
                        if (r > 0) {
                            s.head_got += size_t(r);
                            if (s.head_got == 8) {
                                std::memcpy(&s.want, s.head, 8);
                                if (s.want > (uint64_t(1) << 32)) return fail("process " + std::to_string(peers[i]) + " announced a message of " + std::to_string(s.want) + " bytes");
                                in[i].resize(size_t(s.want));
                                if (s.want == 0) s.rx_done = true;
                            }
                        }
                    } else {
                        r = ::recv(pfs[i].fd, &in[i][s.got], size_t(s.want) - s.got, MSG_DONTWAIT);
                        if (r > 0) { s.got += size_t(r); if (s.got == s.want) s.rx_done = true; }
                    }
                    if (r == 0) return fail("process " + std::to_string(peers[i]) + " closed the connection");
                    if (r < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return fail("receive from process " + std::to_string(peers[i]) + ": " + errno_text());
                }
            }
        }
        for (size_t i = 0; i < peers.size(); ++i) {
            ++stats.messages_sent; stats.bytes_sent += out[i].size() + 8;
            ++stats.messages_received; stats.bytes_received += in[i].size() + 8;
        }
        return true;
    }

    // The same value from every process to every process: returns all of them, indexed by process.
    bool all_gather(const std::string& mine, std::vector<std::string>& all, int timeout_ms) {
        std::vector<uint32_t> peers;
        for (uint32_t p = 0; p < total_; ++p)
            if (p != id_) peers.push_back(p);
        std::vector<std::string> out(peers.size(), mine), in;
        if (!exchange(peers, out, in, timeout_ms)) return false;
        all.assign(total_, std::string());
        all[id_] = mine;
        for (size_t i = 0; i < peers.size(); ++i) all[peers[i]] = std::move(in[i]);
        return true;
    }

    void close_all() {
        for (int& fd : fds_)
            if (fd >= 0) { ::close(fd); fd = -1; }
    }

private:
    uint32_t id_, total_;
    std::string dir_, host_;
    std::vector<int> fds_;

    static long long now_ms() { return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
    static std::string errno_text() { return std::strerror(errno); }
    bool fail(const std::string& what) { error = what; return false; }
    std::string address_file(uint32_t p) const { return dir_ + "/node_" + std::to_string(p) + ".addr"; }
    bool read_address(uint32_t p, std::string& host, int& port) const {
        std::ifstream f(address_file(p));
        std::string line;
        if (!f || !std::getline(f, line)) return false;
        size_t colon = line.rfind(':');
        if (colon == std::string::npos) return false;
        host = line.substr(0, colon);
        port = std::atoi(line.c_str() + colon + 1);
        return port > 0;
    }
    void adopt(uint32_t p, int fd) {
        int one = 1;
        ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
        timeval none{0, 0};
        ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &none, sizeof none);
        fds_[p] = fd;
    }
};

}  // namespace nspice
