// HostTransport: framed TCP full mesh between the ranks of one process group.
//
// Role on B200: GPU tensors never touch it (their data plane is NVLink peer
// memory written from inside the collective kernels).  It carries CPU-tensor
// collectives, point-to-point messages between CPU tensors, heartbeats and
// ABORT propagation.
//
// Receive side is demultiplexed: one reader thread per peer reads frame headers
// and routes each payload by key -- (seq << 32 | tid) for collectives, the user
// tag for send/recv -- straight into the buffer of a posted receive, or, if the
// receive has not been posted yet, into a pooled "parked" buffer that the later
// post_recv drains.  Parked bytes are bounded (park_limit_bytes): a reader that
// hits the bound waits for receivers to drain, and reports a desynchronised
// peer if they do not.  Sends are chunked into frames of at most chunk_bytes.
//
// Failure semantics: EOF or a socket error on a peer fails every receive posted
// to that peer; an ABORT frame from any peer fails every receive on every peer
// and invokes on_abort; send_abort() tells all peers (best effort).
// Parity: reference csrc/transport/Transport.hpp:51-111 and
// csrc/transport/TcpTransport.cpp:203-1127 (behavioural, not structural).
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "runtime/mempool.h"
#include "transport/protocol.h"

namespace mccl {

struct TransportConfig {
  std::string listen_addr = "auto";  // address published to peers
  std::string ifname;                // interface to take the address from
  int port_base = 0;                 // 0: ephemeral port; else try port_base + rank first
  size_t chunk_bytes = 16u << 20;
  bool crc = false;
  int connect_timeout_ms = 30000;
  int recv_timeout_ms = 300000;
  size_t park_limit_bytes = size_t(512) << 20;
  int sock_bufsize = 4 << 20;
  static TransportConfig from_env();
};

class HostTransport {
 public:
  struct Ticket {
    int peer = -1;
    uint64_t key = 0;
    uint8_t* buf = nullptr;
    size_t cap = 0;
    size_t received = 0;
    bool done = false;
    bool reader_busy = false;  // reader is copying into buf right now
    bool cancelled = false;
    uint8_t flags = 0;         // flags of the message that satisfied the receive
    std::string error;
  };
  using TicketPtr = std::shared_ptr<Ticket>;

  HostTransport(int rank, int world_size, TransportConfig cfg);
  ~HostTransport();

  // "ip:port" this rank listens on.
  std::string listen_endpoint() const { return endpoint_; }
  // endpoints[r] = listen_endpoint() of rank r.  Connects to higher ranks,
  // accepts lower ranks, handshakes both ways, starts the readers.
  void connect_all(const std::vector<std::string>& endpoints);

  static uint64_t collective_key(uint32_t seq, uint32_t tid) {
    return (static_cast<uint64_t>(seq) << 32) | tid;
  }
  static uint64_t p2p_key(uint32_t tag) { return (1ull << 63) | tag; }

  void send(int peer, OpType op, uint32_t seq, uint32_t tid, const void* data, size_t nbytes,
            uint8_t extra_flags = 0);
  TicketPtr post_recv(int peer, uint64_t key, void* buf, size_t cap);
  // Blocks until the receive completes; returns the byte count.  Throws
  // TimeoutError / TransportError.  timeout <= 0 uses cfg.recv_timeout_ms.
  size_t wait_recv(const TicketPtr& t, int timeout_ms = 0);
  // post_recv + send + wait in the deadlock-free order.
  size_t send_recv(int peer, OpType op, uint32_t seq, uint32_t send_tid, const void* sbuf,
                   size_t sbytes, uint32_t recv_tid, void* rbuf, size_t rcap);
  void cancel_recvs(uint32_t seq);

  void send_heartbeat();
  void send_abort(const std::string& why);
  bool is_peer_connected(int peer) const;
  bool aborted() const { return aborted_.load(); }
  int64_t ms_since_heard(int peer) const;
  void shutdown();

  uint64_t bytes_sent() const { return bytes_sent_.load(); }
  uint64_t bytes_recv() const { return bytes_recv_.load(); }
  size_t parked_bytes() const { return parked_bytes_.load(); }
  const TransportConfig& config() const { return cfg_; }

  // Called (from a reader thread) when a peer sent ABORT or its link died.
  std::function<void(int peer, const std::string& why)> on_peer_failure;

 private:
  struct Parked {
    PooledBuffer buf;
    size_t size = 0;
    bool complete = false;
    uint8_t flags = 0;
    TicketPtr adopter;
  };
  struct Peer {
    int fd = -1;
    std::atomic<bool> connected{false};
    std::mutex send_mu;
    std::mutex mu;  // guards posted/parked and the tickets routed to this peer
    std::condition_variable cv;
    std::unordered_map<uint64_t, std::deque<TicketPtr>> posted;
    std::unordered_map<uint64_t, std::deque<std::shared_ptr<Parked>>> parked;
    std::string fail_reason;
    std::thread reader;
    std::atomic<int64_t> last_heard_ms{0};
    std::atomic<bool> departed{false};  // peer announced an orderly shutdown
  };

  void reader_loop(int peer);
  void route_payload(int peer, const MessageHeader& h);
  void fail_peer(int peer, const std::string& why, bool notify);
  void fail_all(const std::string& why);
  void send_frame(Peer& p, const MessageHeader& h, const void* payload);
  static uint64_t key_of(const MessageHeader& h);

  int rank_, ws_;
  TransportConfig cfg_;
  int listen_fd_ = -1;
  std::string endpoint_;
  std::vector<std::unique_ptr<Peer>> peers_;
  std::atomic<bool> stopping_{false};
  std::atomic<bool> aborted_{false};
  std::atomic<uint64_t> bytes_sent_{0}, bytes_recv_{0};
  std::atomic<size_t> parked_bytes_{0};
  std::mutex park_mu_;
  std::condition_variable park_cv_;
};

}  // namespace mccl
