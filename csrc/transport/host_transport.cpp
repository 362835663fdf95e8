#include "transport/host_transport.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>

#include "common/env.h"
#include "common/errors.h"
#include "common/log.h"

namespace mccl {

namespace {

int64_t now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

void set_sock_opts(int fd, int bufsize) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  setsockopt(fd, SOL_SOCKET, SO_KEEPALIVE, &one, sizeof(one));
  if (bufsize > 0) {
    setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &bufsize, sizeof(bufsize));
    setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &bufsize, sizeof(bufsize));
  }
}

// Reads exactly n bytes; returns false on EOF/error.
bool recv_all(int fd, void* buf, size_t n) {
  uint8_t* p = static_cast<uint8_t*>(buf);
  while (n > 0) {
    size_t want = std::min<size_t>(n, size_t(1) << 30);
    ssize_t r = ::recv(fd, p, want, 0);
    if (r > 0) {
      p += r;
      n -= static_cast<size_t>(r);
    } else if (r == 0) {
      return false;
    } else if (errno == EINTR) {
      continue;
    } else {
      return false;
    }
  }
  return true;
}

bool send_iov(int fd, struct iovec* iov, int cnt) {
  while (cnt > 0) {
    struct msghdr mh;
    std::memset(&mh, 0, sizeof(mh));
    mh.msg_iov = iov;
    mh.msg_iovlen = cnt;
    ssize_t w = ::sendmsg(fd, &mh, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    size_t left = static_cast<size_t>(w);
    while (cnt > 0 && left >= iov->iov_len) {
      left -= iov->iov_len;
      ++iov;
      --cnt;
    }
    if (cnt > 0 && left > 0) {
      iov->iov_base = static_cast<uint8_t*>(iov->iov_base) + left;
      iov->iov_len -= left;
    }
  }
  return true;
}

std::string local_addr_towards(const std::string& host, int port) {
  // UDP "connect" picks the outgoing interface without sending anything.
  struct addrinfo hints, *res = nullptr;
  std::memset(&hints, 0, sizeof(hints));
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_DGRAM;
  if (getaddrinfo(host.c_str(), std::to_string(port > 0 ? port : 9).c_str(), &hints, &res) != 0 ||
      !res)
    return "";
  std::string out;
  int fd = ::socket(AF_INET, SOCK_DGRAM, 0);
  if (fd >= 0) {
    if (::connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
      struct sockaddr_in sa;
      socklen_t sl = sizeof(sa);
      if (getsockname(fd, reinterpret_cast<struct sockaddr*>(&sa), &sl) == 0) {
        char buf[INET_ADDRSTRLEN];
        if (inet_ntop(AF_INET, &sa.sin_addr, buf, sizeof(buf))) out = buf;
      }
    }
    ::close(fd);
  }
  freeaddrinfo(res);
  return out;
}

std::string addr_of_interface(const std::string& ifname) {
  struct ifaddrs* ifa = nullptr;
  std::string out;
  if (getifaddrs(&ifa) != 0) return out;
  for (auto* p = ifa; p; p = p->ifa_next) {
    if (!p->ifa_addr || p->ifa_addr->sa_family != AF_INET) continue;
    if (ifname != p->ifa_name) continue;
    char buf[INET_ADDRSTRLEN];
    auto* sa = reinterpret_cast<struct sockaddr_in*>(p->ifa_addr);
    if (inet_ntop(AF_INET, &sa->sin_addr, buf, sizeof(buf))) out = buf;
    break;
  }
  freeifaddrs(ifa);
  return out;
}

}  // namespace

TransportConfig TransportConfig::from_env() {
  TransportConfig c;
  c.listen_addr = env_str("MCCL_LISTEN_ADDR", "auto");
  c.ifname = env_str("MCCL_IFNAME", "");
  // An explicit MCCL_PORT_BASE pins ports to base+rank; otherwise the kernel
  // picks a free port and the endpoint travels through the Store.
  c.port_base = static_cast<int>(env_int("MCCL_PORT_BASE", 0));
  c.chunk_bytes = static_cast<size_t>(std::max<int64_t>(env_int("MCCL_CHUNK_BYTES", 16 << 20), 1));
  c.crc = env_bool("MCCL_TRANSPORT_CRC", false);
  c.connect_timeout_ms = static_cast<int>(env_int("MCCL_CONNECT_TIMEOUT_MS", 30000));
  c.recv_timeout_ms = static_cast<int>(
      env_int("MCCL_RECV_TIMEOUT_MS", env_int("MCCL_WATCHDOG_TIMEOUT_MS", 300000)));
  c.park_limit_bytes = static_cast<size_t>(
      std::clamp<int64_t>(env_int("MCCL_DEMUX_PARK_BYTES", 512ll << 20), 1 << 16, 4ll << 30));
  c.sock_bufsize = static_cast<int>(env_int("MCCL_SOCK_BUFSIZE", 4 << 20));
  if (env_str("MCCL_LINK_PROFILE", "") == "thunderbolt") {
    // High-bandwidth-link preset: larger socket buffers, at least 16 MiB frames.
    c.sock_bufsize = std::max(c.sock_bufsize, 32 << 20);
    c.chunk_bytes = std::max<size_t>(c.chunk_bytes, 16u << 20);
  }
  return c;
}

HostTransport::HostTransport(int rank, int world_size, TransportConfig cfg)
    : rank_(rank), ws_(world_size), cfg_(std::move(cfg)) {
  for (int i = 0; i < ws_; ++i) peers_.emplace_back(new Peer());

  listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
  MCCL_CHECK_TRANSPORT(listen_fd_ >= 0, "socket(): " << std::strerror(errno));
  int one = 1;
  setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));

  struct sockaddr_in sa;
  std::memset(&sa, 0, sizeof(sa));
  sa.sin_family = AF_INET;
  sa.sin_addr.s_addr = htonl(INADDR_ANY);
  bool bound = false;
  if (cfg_.port_base > 0 && cfg_.port_base + rank_ <= 65535) {
    sa.sin_port = htons(static_cast<uint16_t>(cfg_.port_base + rank_));
    bound = ::bind(listen_fd_, reinterpret_cast<struct sockaddr*>(&sa), sizeof(sa)) == 0;
    if (!bound)
      MCCL_WARN("port %d (MCCL_PORT_BASE+rank) is taken: %s; using an ephemeral port",
                cfg_.port_base + rank_, std::strerror(errno));
  }
  if (!bound) {
    sa.sin_port = 0;
    MCCL_CHECK_TRANSPORT(
        ::bind(listen_fd_, reinterpret_cast<struct sockaddr*>(&sa), sizeof(sa)) == 0,
        "bind(): " << std::strerror(errno));
  }
  MCCL_CHECK_TRANSPORT(::listen(listen_fd_, std::max(16, ws_ * 2)) == 0,
                       "listen(): " << std::strerror(errno));
  socklen_t sl = sizeof(sa);
  getsockname(listen_fd_, reinterpret_cast<struct sockaddr*>(&sa), &sl);
  int port = ntohs(sa.sin_port);

  std::string addr;
  if (!cfg_.listen_addr.empty() && cfg_.listen_addr != "auto") {
    addr = cfg_.listen_addr;
  } else if (!cfg_.ifname.empty()) {
    addr = addr_of_interface(cfg_.ifname);
    if (addr.empty()) MCCL_WARN("MCCL_IFNAME=%s has no IPv4 address", cfg_.ifname.c_str());
  }
  if (addr.empty()) {
    std::string master = env_str("MASTER_ADDR", "127.0.0.1");
    if (master == "localhost" || master.rfind("127.", 0) == 0) {
      addr = "127.0.0.1";
    } else {
      addr = local_addr_towards(master, static_cast<int>(env_int("MASTER_PORT", 29500)));
      if (addr.empty()) {
        MCCL_WARN("could not resolve MASTER_ADDR=%s; publishing 127.0.0.1", master.c_str());
        addr = "127.0.0.1";
      }
    }
  }
  endpoint_ = addr + ":" + std::to_string(port);
  MCCL_DEBUG("rank %d listening on %s", rank_, endpoint_.c_str());
}

HostTransport::~HostTransport() { shutdown(); }

uint64_t HostTransport::key_of(const MessageHeader& h) {
  if (h.op == static_cast<uint8_t>(OpType::SEND) || h.op == static_cast<uint8_t>(OpType::RECV))
    return p2p_key(h.tid);
  return collective_key(h.seq, h.tid);
}

void HostTransport::connect_all(const std::vector<std::string>& endpoints) {
  MCCL_CHECK_TRANSPORT(static_cast<int>(endpoints.size()) == ws_, "endpoint list size mismatch");
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(cfg_.connect_timeout_ms);

  HandshakePayload mine;
  std::memset(&mine, 0, sizeof(mine));
  mine.version = MCCL_PROTOCOL_VERSION;
  mine.rank = static_cast<uint32_t>(rank_);
  mine.world_size = static_cast<uint32_t>(ws_);
  gethostname(mine.hostname, sizeof(mine.hostname) - 1);

  auto send_hs = [&](int fd) {
    MessageHeader h = make_header(OpType::HANDSHAKE, 0, 0, 0, sizeof(mine), FLAG_LAST_CHUNK);
    struct iovec iov[2] = {{&h, sizeof(h)}, {&mine, sizeof(mine)}};
    return send_iov(fd, iov, 2);
  };
  auto recv_hs = [&](int fd, HandshakePayload& out) {
    MessageHeader h;
    if (!recv_all(fd, &h, sizeof(h))) return false;
    if (h.version != MCCL_PROTOCOL_VERSION || h.op != static_cast<uint8_t>(OpType::HANDSHAKE) ||
        h.payload_bytes != sizeof(HandshakePayload))
      throw ProtocolError("bad handshake frame (version " + std::to_string(h.version) + ")");
    return recv_all(fd, &out, sizeof(out));
  };
  auto validate = [&](const HandshakePayload& hs, int expect_rank) {
    if (hs.version != MCCL_PROTOCOL_VERSION)
      throw ProtocolError("peer speaks protocol " + std::to_string(hs.version) + ", expected " +
                          std::to_string(MCCL_PROTOCOL_VERSION));
    if (static_cast<int>(hs.world_size) != ws_)
      throw ProtocolError("peer world_size " + std::to_string(hs.world_size) + " != " +
                          std::to_string(ws_));
    if (static_cast<int>(hs.rank) >= ws_ || (expect_rank >= 0 && static_cast<int>(hs.rank) != expect_rank))
      throw ProtocolError("unexpected peer rank " + std::to_string(hs.rank));
  };

  // Accept lower ranks on a helper thread while connecting to higher ranks.
  std::string accept_err;
  std::thread acceptor([&] {
    try {
      int need = rank_;
      while (need > 0) {
        struct pollfd pfd = {listen_fd_, POLLIN, 0};
        auto left = std::chrono::duration_cast<std::chrono::milliseconds>(
                        deadline - std::chrono::steady_clock::now())
                        .count();
        if (left <= 0) throw TransportError("timed out accepting lower ranks");
        int pr = ::poll(&pfd, 1, static_cast<int>(std::min<int64_t>(left, 500)));
        if (pr <= 0) continue;
        int fd = ::accept(listen_fd_, nullptr, nullptr);
        if (fd < 0) continue;
        set_sock_opts(fd, cfg_.sock_bufsize);
        HandshakePayload hs;
        if (!recv_hs(fd, hs)) {
          ::close(fd);
          continue;
        }
        validate(hs, -1);
        int pr_rank = static_cast<int>(hs.rank);
        if (pr_rank >= rank_ || peers_[pr_rank]->fd >= 0) {
          ::close(fd);
          throw ProtocolError("duplicate or out-of-order connection from rank " +
                              std::to_string(pr_rank));
        }
        if (!send_hs(fd)) {
          ::close(fd);
          throw TransportError("handshake reply failed");
        }
        peers_[pr_rank]->fd = fd;
        peers_[pr_rank]->connected = true;
        --need;
      }
    } catch (const std::exception& e) {
      accept_err = e.what();
    }
  });

  std::string connect_err;
  try {
    for (int p = rank_ + 1; p < ws_; ++p) {
      const std::string& ep = endpoints[p];
      auto colon = ep.rfind(':');
      MCCL_CHECK_TRANSPORT(colon != std::string::npos, "bad endpoint '" << ep << "'");
      std::string host = ep.substr(0, colon), port = ep.substr(colon + 1);
      int fd = -1;
      for (;;) {
        struct addrinfo hints, *res = nullptr;
        std::memset(&hints, 0, sizeof(hints));
        hints.ai_family = AF_INET;
        hints.ai_socktype = SOCK_STREAM;
        if (getaddrinfo(host.c_str(), port.c_str(), &hints, &res) == 0 && res) {
          fd = ::socket(AF_INET, SOCK_STREAM, 0);
          if (fd >= 0) {
            if (::connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
              freeaddrinfo(res);
              break;
            }
            ::close(fd);
            fd = -1;
          }
          freeaddrinfo(res);
        }
        if (std::chrono::steady_clock::now() > deadline)
          throw TransportError("timed out connecting to rank " + std::to_string(p) + " at " + ep);
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
      }
      set_sock_opts(fd, cfg_.sock_bufsize);
      HandshakePayload hs;
      if (!send_hs(fd) || !recv_hs(fd, hs)) {
        ::close(fd);
        throw TransportError("handshake with rank " + std::to_string(p) + " failed");
      }
      validate(hs, p);
      peers_[p]->fd = fd;
      peers_[p]->connected = true;
    }
  } catch (const std::exception& e) {
    connect_err = e.what();
  }
  acceptor.join();
  if (!connect_err.empty()) throw TransportError(connect_err);
  if (!accept_err.empty()) throw TransportError(accept_err);

  int64_t t = now_ms();
  for (int p = 0; p < ws_; ++p) {
    if (p == rank_) continue;
    peers_[p]->last_heard_ms = t;
    peers_[p]->reader = std::thread([this, p] { reader_loop(p); });
  }
  MCCL_DEBUG("rank %d: host mesh of %d ranks connected", rank_, ws_);
}

void HostTransport::send_frame(Peer& p, const MessageHeader& h, const void* payload) {
  struct iovec iov[2];
  iov[0].iov_base = const_cast<MessageHeader*>(&h);
  iov[0].iov_len = sizeof(h);
  int cnt = 1;
  if (h.payload_bytes > 0) {
    iov[1].iov_base = const_cast<void*>(payload);
    iov[1].iov_len = h.payload_bytes;
    cnt = 2;
  }
  if (!send_iov(p.fd, iov, cnt)) throw TransportError(std::string("send failed: ") + std::strerror(errno));
  bytes_sent_ += sizeof(h) + h.payload_bytes;
}

void HostTransport::send(int peer, OpType op, uint32_t seq, uint32_t tid, const void* data,
                         size_t nbytes, uint8_t extra_flags) {
  MCCL_CHECK_TRANSPORT(peer >= 0 && peer < ws_ && peer != rank_, "bad peer " << peer);
  Peer& p = *peers_[peer];
  if (aborted_.load()) throw TransportError("transport aborted");
  if (!p.connected.load()) throw TransportError("peer " + std::to_string(peer) + " is not connected");
  const uint8_t* src = static_cast<const uint8_t*>(data);
  size_t off = 0;
  uint32_t idx = 0;
  // The send lock is held for the whole message so that its frames are
  // contiguous on the stream (the reader relies on that for parked messages).
  std::lock_guard<std::mutex> g(p.send_mu);
  do {
    size_t n = std::min(cfg_.chunk_bytes, nbytes - off);
    uint8_t flags = extra_flags;
    if (off + n >= nbytes) flags |= FLAG_LAST_CHUNK;
    uint32_t crc = 0;
    if (cfg_.crc && n > 0) {
      flags |= FLAG_HAS_CRC;
      crc = crc32_compute(src + off, n);
    }
    MessageHeader h = make_header(op, seq, tid, idx, static_cast<uint32_t>(n), flags, crc);
    send_frame(p, h, src + off);
    off += n;
    ++idx;
  } while (off < nbytes);
}

HostTransport::TicketPtr HostTransport::post_recv(int peer, uint64_t key, void* buf, size_t cap) {
  MCCL_CHECK_TRANSPORT(peer >= 0 && peer < ws_ && peer != rank_, "bad peer " << peer);
  Peer& p = *peers_[peer];
  auto t = std::make_shared<Ticket>();
  t->peer = peer;
  t->key = key;
  t->buf = static_cast<uint8_t*>(buf);
  t->cap = cap;
  std::unique_lock<std::mutex> lk(p.mu);
  auto pit = p.parked.find(key);
  if (pit != p.parked.end() && !pit->second.empty()) {
    // Find the first parked message nobody has adopted yet.
    for (auto it = pit->second.begin(); it != pit->second.end(); ++it) {
      auto pk = *it;
      if (pk->adopter) continue;
      if (pk->complete) {
        if (pk->size > cap) {
          t->error = "parked message of " + std::to_string(pk->size) + " bytes exceeds receive buffer of " +
                     std::to_string(cap);
        } else {
          if (pk->size) std::memcpy(t->buf, pk->buf.data(), pk->size);
          t->received = pk->size;
          t->flags = pk->flags;
        }
        t->done = true;
        size_t freed = pk->size;
        pit->second.erase(it);
        if (pit->second.empty()) p.parked.erase(pit);
        lk.unlock();
        parked_bytes_ -= freed;
        park_cv_.notify_all();
        return t;
      }
      pk->adopter = t;  // still arriving: the reader hands it over when complete
      return t;
    }
  }
  if (!p.connected.load() || aborted_.load()) {
    t->error = aborted_.load() ? "transport aborted"
                               : ("peer " + std::to_string(peer) + " disconnected: " + p.fail_reason);
    t->done = true;
    return t;
  }
  p.posted[key].push_back(t);
  lk.unlock();
  p.cv.notify_all();  // a reader may be holding a large frame back for exactly this receive
  return t;
}

size_t HostTransport::wait_recv(const TicketPtr& t, int timeout_ms) {
  Peer& p = *peers_[t->peer];
  if (timeout_ms <= 0) timeout_ms = cfg_.recv_timeout_ms;
  std::unique_lock<std::mutex> lk(p.mu);
  bool ok = p.cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return t->done; });
  if (!ok) {
    // Withdraw the ticket; never free the caller's buffer under a running copy.
    t->cancelled = true;
    p.cv.wait(lk, [&] { return !t->reader_busy; });
    auto it = p.posted.find(t->key);
    if (it != p.posted.end()) {
      auto& dq = it->second;
      dq.erase(std::remove(dq.begin(), dq.end(), t), dq.end());
      if (dq.empty()) p.posted.erase(it);
    }
    throw TimeoutError("receive from rank " + std::to_string(t->peer) + " timed out after " +
                       std::to_string(timeout_ms) + " ms");
  }
  if (!t->error.empty()) throw TransportError(t->error);
  return t->received;
}

size_t HostTransport::send_recv(int peer, OpType op, uint32_t seq, uint32_t send_tid,
                                const void* sbuf, size_t sbytes, uint32_t recv_tid, void* rbuf,
                                size_t rcap) {
  auto t = post_recv(peer, collective_key(seq, recv_tid), rbuf, rcap);
  send(peer, op, seq, send_tid, sbuf, sbytes);
  return wait_recv(t);
}

void HostTransport::cancel_recvs(uint32_t seq) {
  for (int pr = 0; pr < ws_; ++pr) {
    if (pr == rank_) continue;
    Peer& p = *peers_[pr];
    std::unique_lock<std::mutex> lk(p.mu);
    for (auto it = p.posted.begin(); it != p.posted.end();) {
      uint64_t key = it->first;
      bool is_p2p = (key >> 63) != 0;
      if (!is_p2p && static_cast<uint32_t>(key >> 32) == seq) {
        for (auto& t : it->second) {
          t->cancelled = true;
          p.cv.wait(lk, [&] { return !t->reader_busy; });
          if (!t->done) {
            t->error = "receive cancelled";
            t->done = true;
          }
        }
        it = p.posted.erase(it);
      } else {
        ++it;
      }
    }
    p.cv.notify_all();
  }
}

void HostTransport::fail_peer(int peer, const std::string& why, bool notify) {
  Peer& p = *peers_[peer];
  {
    std::lock_guard<std::mutex> g(p.mu);
    p.connected = false;
    if (p.fail_reason.empty()) p.fail_reason = why;
    for (auto& kv : p.posted)
      for (auto& t : kv.second)
        if (!t->done) {
          t->error = "peer " + std::to_string(peer) + ": " + why;
          t->done = true;
        }
    p.posted.clear();
    for (auto& kv : p.parked)
      for (auto& pk : kv.second)
        if (pk->adopter && !pk->adopter->done) {
          pk->adopter->error = "peer " + std::to_string(peer) + ": " + why;
          pk->adopter->done = true;
        }
    p.cv.notify_all();
  }
  if (notify && !stopping_.load() && on_peer_failure) on_peer_failure(peer, why);
}

void HostTransport::fail_all(const std::string& why) {
  for (int pr = 0; pr < ws_; ++pr) {
    if (pr == rank_) continue;
    Peer& p = *peers_[pr];
    std::lock_guard<std::mutex> g(p.mu);
    for (auto& kv : p.posted)
      for (auto& t : kv.second)
        if (!t->done) {
          t->error = why;
          t->done = true;
        }
    p.posted.clear();
    p.cv.notify_all();
  }
}

namespace {
constexpr size_t kParkGraceBytes = 256 << 10;
constexpr int kParkGraceMs = 3;
}  // namespace

void HostTransport::route_payload(int peer, const MessageHeader& h) {
  Peer& p = *peers_[peer];
  const uint64_t key = key_of(h);
  const size_t n = h.payload_bytes;
  const bool last = (h.flags & FLAG_LAST_CHUNK) != 0;

  TicketPtr ticket;
  std::shared_ptr<Parked> park;
  uint8_t* dst = nullptr;
  {
    std::unique_lock<std::mutex> lk(p.mu);
    bool waited_for_space = false, grace_done = false;
    for (;;) {
      // 1. continuation of a message that is already being parked
      auto pit = p.parked.find(key);
      if (pit != p.parked.end() && !pit->second.empty() && !pit->second.back()->complete) {
        park = pit->second.back();
        break;
      }
      // 2. a posted receive
      auto it = p.posted.find(key);
      if (it != p.posted.end()) {
        while (!it->second.empty() && (it->second.front()->done || it->second.front()->cancelled))
          it->second.pop_front();
        if (!it->second.empty()) ticket = it->second.front();
        if (it->second.empty()) p.posted.erase(it);
      }
      if (ticket) break;
      // 3. no receive yet.  A large frame is worth a short grace period: in back-to-back
      // collectives the sender runs a little ahead of the receiver's next post, and parking
      // costs a pooled buffer plus a second copy of the whole payload.
      if (!grace_done && n >= kParkGraceBytes) {
        grace_done = true;
        p.cv.wait_for(lk, std::chrono::milliseconds(kParkGraceMs), [&] {
          auto q = p.posted.find(key);
          return stopping_.load() || aborted_.load() || (q != p.posted.end() && !q->second.empty());
        });
        continue;
      }
      // 4. park it.  Waiting for park space drops the lock, so a receive may be
      // posted meanwhile: look again before creating the parked message.
      if (!waited_for_space) {
        lk.unlock();
        {
          std::unique_lock<std::mutex> pl(park_mu_);
          bool ok = park_cv_.wait_for(pl, std::chrono::milliseconds(cfg_.recv_timeout_ms), [&] {
            return stopping_.load() || parked_bytes_.load() + n <= cfg_.park_limit_bytes ||
                   parked_bytes_.load() == 0;
          });
          if (!ok)
            throw ProtocolError("parked-message limit of " + std::to_string(cfg_.park_limit_bytes) +
                                " bytes exceeded: ranks are desynchronised");
        }
        lk.lock();
        waited_for_space = true;
        continue;
      }
      park = std::make_shared<Parked>();
      p.parked[key].push_back(park);
      break;
    }
    if (ticket) {
      if (ticket->received + n > ticket->cap) {
        ticket->error = "message longer than the posted receive (" +
                        std::to_string(ticket->received + n) + " > " + std::to_string(ticket->cap) + ")";
        ticket->done = true;
        p.cv.notify_all();
        throw ProtocolError(ticket->error);
      }
      ticket->reader_busy = true;
      dst = ticket->buf + ticket->received;
    } else {
      size_t need = park->size + n;
      if (need > park->buf.capacity()) {
        PooledBuffer bigger = staging_memory_pool().acquire(std::max(need, park->buf.capacity() * 2));
        if (park->size) std::memcpy(bigger.data(), park->buf.data(), park->size);
        park->buf = std::move(bigger);
      }
      dst = park->buf.as<uint8_t>() + park->size;
    }
  }

  bool ok = n == 0 || recv_all(p.fd, dst, n);
  bool crc_ok = true;
  if (ok && (h.flags & FLAG_HAS_CRC) && n > 0) crc_ok = crc32_compute(dst, n) == h.crc;
  bytes_recv_ += sizeof(h) + n;

  std::unique_lock<std::mutex> lk(p.mu);
  if (ticket) {
    ticket->reader_busy = false;
    if (!ok || !crc_ok) {
      ticket->error = ok ? "CRC mismatch" : "connection closed mid-message";
      ticket->done = true;
    } else {
      ticket->received += n;
      if (last) {
        ticket->flags = h.flags;
        ticket->done = true;
        auto it = p.posted.find(key);
        if (it != p.posted.end()) {
          auto& dq = it->second;
          dq.erase(std::remove(dq.begin(), dq.end(), ticket), dq.end());
          if (dq.empty()) p.posted.erase(it);
        }
      }
    }
    p.cv.notify_all();
  } else {
    if (ok && crc_ok) {
      park->size += n;
      parked_bytes_ += n;
      if (last) {
        park->complete = true;
        park->flags = h.flags;
        if (park->adopter) {
          TicketPtr t = park->adopter;
          if (!t->cancelled) {
            if (park->size > t->cap) {
              t->error = "parked message exceeds receive buffer";
            } else {
              if (park->size) std::memcpy(t->buf, park->buf.data(), park->size);
              t->received = park->size;
              t->flags = park->flags;
            }
            t->done = true;
          }
          auto& dq = p.parked[key];
          dq.erase(std::remove(dq.begin(), dq.end(), park), dq.end());
          if (dq.empty()) p.parked.erase(key);
          parked_bytes_ -= park->size;
          park_cv_.notify_all();
          p.cv.notify_all();
        }
      }
    }
  }
  lk.unlock();
  if (!ok) throw TransportError("connection closed mid-message");
  if (!crc_ok) throw ProtocolError("CRC mismatch on frame from rank " + std::to_string(peer));
}

void HostTransport::reader_loop(int peer) {
  Peer& p = *peers_[peer];
  std::string why;
  bool notify = true;
  try {
    for (;;) {
      MessageHeader h;
      if (!recv_all(p.fd, &h, sizeof(h))) {
        why = "connection closed";
        break;
      }
      p.last_heard_ms = now_ms();
      if (h.version != MCCL_PROTOCOL_VERSION)
        throw ProtocolError("frame with protocol version " + std::to_string(h.version));
      if (h.op == static_cast<uint8_t>(OpType::HEARTBEAT)) {
        bytes_recv_ += sizeof(h);
        if (h.flags & FLAG_GOODBYE) p.departed = true;
        continue;
      }
      if (h.op == static_cast<uint8_t>(OpType::ABORT)) {
        std::string msg(h.payload_bytes, '\0');
        if (h.payload_bytes && !recv_all(p.fd, msg.data(), h.payload_bytes)) msg = "(truncated)";
        aborted_ = true;
        why = "ABORT from rank " + std::to_string(peer) + ": " + msg;
        fail_all(why);
        break;
      }
      route_payload(peer, h);
    }
  } catch (const std::exception& e) {
    why = e.what();
  }
  if (stopping_.load()) notify = false;
  if (p.departed.load()) {  // orderly shutdown of the peer: not a failure of this group
    notify = false;
    why = "peer shut down";
  }
  fail_peer(peer, why.empty() ? "reader stopped" : why, notify);
}

void HostTransport::send_heartbeat() {
  for (int pr = 0; pr < ws_; ++pr) {
    if (pr == rank_) continue;
    Peer& p = *peers_[pr];
    if (!p.connected.load()) continue;
    MessageHeader h = make_header(OpType::HEARTBEAT, 0, 0, 0, 0, FLAG_LAST_CHUNK);
    std::unique_lock<std::mutex> g(p.send_mu, std::try_to_lock);
    if (!g.owns_lock()) continue;  // a data send is in progress: the link is evidently alive
    try {
      send_frame(p, h, nullptr);
    } catch (...) {
    }
  }
}

void HostTransport::send_abort(const std::string& why) {
  aborted_ = true;
  std::string msg = why.substr(0, 1024);
  for (int pr = 0; pr < ws_; ++pr) {
    if (pr == rank_) continue;
    Peer& p = *peers_[pr];
    if (!p.connected.load()) continue;
    MessageHeader h = make_header(OpType::ABORT, 0, 0, 0, static_cast<uint32_t>(msg.size()), FLAG_LAST_CHUNK);
    // Bounded attempt: a peer stuck in a long send must not block abort delivery forever.
    std::unique_lock<std::mutex> g(p.send_mu, std::defer_lock);
    bool got = false;
    for (int i = 0; i < 200 && !(got = g.try_lock()); ++i)
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    if (!got) continue;
    try {
      send_frame(p, h, msg.data());
    } catch (...) {
    }
  }
  fail_all("transport aborted: " + why);
}

bool HostTransport::is_peer_connected(int peer) const {
  if (peer == rank_) return true;
  if (peer < 0 || peer >= ws_) return false;
  return peers_[peer]->connected.load();
}

int64_t HostTransport::ms_since_heard(int peer) const {
  if (peer == rank_ || peer < 0 || peer >= ws_) return 0;
  return now_ms() - peers_[peer]->last_heard_ms.load();
}

void HostTransport::shutdown() {
  bool e = false;
  if (!stopping_.compare_exchange_strong(e, true)) return;
  park_cv_.notify_all();
  // 0. tell peers this is an orderly shutdown, so the EOF that follows is not reported as a failure
  for (int pr = 0; pr < ws_; ++pr) {
    if (pr == rank_) continue;
    Peer& p = *peers_[pr];
    if (p.fd < 0 || !p.connected.load()) continue;
    MessageHeader h = make_header(OpType::HEARTBEAT, 0, 0, 0, 0, FLAG_LAST_CHUNK | FLAG_GOODBYE);
    std::unique_lock<std::mutex> g(p.send_mu, std::try_to_lock);
    if (!g.owns_lock()) continue;
    try {
      send_frame(p, h, nullptr);
    } catch (...) {
    }
  }
  // 1. stop accepting, 2. half-close so peers see EOF, 3. join readers and close.
  if (listen_fd_ >= 0) {
    ::close(listen_fd_);
    listen_fd_ = -1;
  }
  for (int pr = 0; pr < ws_; ++pr) {
    Peer& p = *peers_[pr];
    if (p.fd >= 0) ::shutdown(p.fd, SHUT_RDWR);
  }
  for (int pr = 0; pr < ws_; ++pr) {
    Peer& p = *peers_[pr];
    if (p.reader.joinable()) p.reader.join();
    if (p.fd >= 0) {
      ::close(p.fd);
      p.fd = -1;
    }
  }
}

}  // namespace mccl
