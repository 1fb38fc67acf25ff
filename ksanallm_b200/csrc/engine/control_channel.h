// Host-side control plane between the nodes of a multi-node deployment: one master, N-1 workers
// over TCP with a small framed protocol. Provides node registration, barrier, layer-range
// assignment, the minimum-block-count consensus, broadcast of serialized step plans, heartbeats
// with failure detection, and cluster shutdown.
//
// Behavioural counterpart of src/ksana_llm/distributed/control_channel.cpp:63-759,
// raw_socket.cpp:79-407 and distributed_coordinator.cpp:36-104. Everything here is host code; a
// lost peer is detected by socket EOF or missed heartbeats and reported through `alive()` / the
// failure list - device work is never involved in failure handling.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace pybind11 { class module_; }

namespace ksana {

enum PacketType : uint16_t {
  PKT_ADD_NODE = 1, PKT_ADD_NODE_ACK, PKT_BARRIER_REQ, PKT_BARRIER_RSP, PKT_LAYER_REQ, PKT_LAYER_RSP,
  PKT_BLOCKNUM_REQ, PKT_BLOCKNUM_RSP, PKT_SCHEDULE, PKT_HEARTBEAT_REQ, PKT_HEARTBEAT_RSP, PKT_SHUTDOWN,
  PKT_DATA,
};
constexpr uint16_t kPacketMagic = 0x2ea9;

struct Packet {
  uint16_t type = 0;
  int32_t node_rank = 0;
  std::string payload;
};

// Blocking framed socket helpers (return false on EOF / error / timeout).
bool SendPacket(int fd, const Packet& p);
bool RecvPacket(int fd, Packet* p, int timeout_ms);
int ListenOn(const std::string& host, int port, int* bound_port);
int ConnectTo(const std::string& host, int port, int retry_ms);

// Contiguous layer ranges: quotient layers each, the first `remainder` nodes take one more.
std::vector<std::pair<int, int>> SplitLayers(int num_layers, int world_size);

class ControlMaster {
 public:
  ControlMaster(const std::string& host, int port, int world_size, int heartbeat_interval_ms = 30000,
                int heartbeat_timeout_ms = 120000);
  ~ControlMaster();
  int port() const { return port_; }
  bool WaitForNodes(int timeout_ms);               // all workers registered
  bool Barrier(int timeout_ms);
  // Returns this node's range; workers receive theirs. Empty vector on timeout.
  std::vector<std::pair<int, int>> AssignLayers(int num_layers, int timeout_ms);
  int SyncBlockNum(int my_blocks, int timeout_ms); // min over nodes, -1 on timeout
  bool Broadcast(const std::string& bytes);        // serialized step plan to every worker
  void ShutdownCluster();
  bool alive() const { return alive_.load(); }
  std::vector<int> FailedNodes();
  void Stop();

 private:
  struct Peer { int fd = -1; int rank = -1; int64_t last_seen_ms = 0; std::thread reader; bool failed = false; };
  void AcceptLoop();
  void ReaderLoop(Peer* peer);
  void HeartbeatLoop();
  bool Collect(uint16_t type, int timeout_ms, std::map<int, std::string>* values);
  void Reply(uint16_t type, const std::map<int, std::string>& per_rank, const std::string& common);
  void MarkFailed(Peer* p);

  int listen_fd_ = -1, port_ = 0, world_size_;
  int hb_interval_ms_, hb_timeout_ms_;
  std::atomic<bool> alive_{true}, stop_{false};
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<Peer*> peers_;
  std::map<uint16_t, std::map<int, std::string>> pending_;   // request type -> rank -> payload
  std::thread accept_thread_, hb_thread_;
};

class ControlWorker {
 public:
  ControlWorker(const std::string& master_host, int master_port, int node_rank, int heartbeat_interval_ms = 30000,
                int heartbeat_timeout_ms = 120000);
  ~ControlWorker();
  bool Connect(int retry_ms);
  bool Barrier(int timeout_ms);
  std::pair<int, int> GetLayers(int timeout_ms);   // (-1,-1) on timeout
  int SyncBlockNum(int my_blocks, int timeout_ms);
  bool RecvBroadcast(std::string* bytes, int timeout_ms);
  bool alive() const { return alive_.load(); }
  bool shutdown_requested() const { return shutdown_.load(); }
  void Stop();

 private:
  void ReaderLoop();
  void HeartbeatLoop();
  bool Request(uint16_t req, uint16_t rsp, const std::string& payload, std::string* out, int timeout_ms);

  std::string host_;
  int port_, rank_, fd_ = -1;
  int hb_interval_ms_, hb_timeout_ms_;
  std::atomic<bool> alive_{false}, stop_{false}, shutdown_{false};
  std::atomic<int64_t> last_seen_ms_{0};
  std::mutex mu_, send_mu_;
  std::condition_variable cv_;
  std::map<uint16_t, std::deque<std::string>> inbox_;
  std::thread reader_, hb_thread_;
};

void BindControlChannel(pybind11::module_& m);

}  // namespace ksana
