#include "control_channel.h"
#include "logger.h"

#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#ifndef KSANA_NO_PYBIND
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#endif
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>

#include "common.h"

namespace ksana {

namespace {

bool SendAll(int fd, const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n > 0) {
    const ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w <= 0) return false;
    p += w;
    n -= static_cast<size_t>(w);
  }
  return true;
}

bool RecvAll(int fd, void* buf, size_t n, int timeout_ms) {
  char* p = static_cast<char*>(buf);
  const int64_t deadline = timeout_ms < 0 ? -1 : NowMs() + timeout_ms;
  while (n > 0) {
    struct pollfd pfd{fd, POLLIN, 0};
    const int wait = deadline < 0 ? 1000 : static_cast<int>(std::max<int64_t>(0, deadline - NowMs()));
    const int pr = ::poll(&pfd, 1, wait);
    if (pr < 0) return false;
    if (pr == 0) {
      if (deadline >= 0 && NowMs() >= deadline) return false;
      continue;
    }
    const ssize_t r = ::recv(fd, p, n, 0);
    if (r <= 0) return false;   // EOF or error
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

struct Header { uint16_t magic; uint16_t type; uint32_t len; int32_t rank; };

std::string EncodeInts(const std::vector<int>& v) {
  return std::string(reinterpret_cast<const char*>(v.data()), v.size() * sizeof(int));
}
std::vector<int> DecodeInts(const std::string& s) {
  std::vector<int> v(s.size() / sizeof(int));
  std::memcpy(v.data(), s.data(), v.size() * sizeof(int));
  return v;
}

}  // namespace

bool SendPacket(int fd, const Packet& p) {
  Header h{kPacketMagic, p.type, static_cast<uint32_t>(p.payload.size()), p.node_rank};
  return SendAll(fd, &h, sizeof(h)) && (p.payload.empty() || SendAll(fd, p.payload.data(), p.payload.size()));
}

bool RecvPacket(int fd, Packet* p, int timeout_ms) {
  Header h;
  if (!RecvAll(fd, &h, sizeof(h), timeout_ms)) return false;
  if (h.magic != kPacketMagic || h.len > (1u << 30)) return false;
  p->type = h.type;
  p->node_rank = h.rank;
  p->payload.resize(h.len);
  return h.len == 0 || RecvAll(fd, &p->payload[0], h.len, timeout_ms < 0 ? -1 : std::max(timeout_ms, 1000));
}

int ListenOn(const std::string& host, int port, int* bound_port) {
  const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  int one = 1;
  ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (host.empty() || host == "0.0.0.0") addr.sin_addr.s_addr = INADDR_ANY;
  else ::inet_pton(AF_INET, host.c_str(), &addr.sin_addr);
  if (::bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(fd, 64) != 0) {
    ::close(fd);
    return -1;
  }
  socklen_t len = sizeof(addr);
  ::getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len);
  if (bound_port) *bound_port = ntohs(addr.sin_port);
  return fd;
}

int ConnectTo(const std::string& host, int port, int retry_ms) {
  const int64_t deadline = NowMs() + retry_ms;
  do {
    const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return -1;
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(static_cast<uint16_t>(port));
    if (::inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) {
      hostent* he = ::gethostbyname(host.c_str());
      if (!he) { ::close(fd); return -1; }
      std::memcpy(&addr.sin_addr, he->h_addr_list[0], sizeof(addr.sin_addr));
    }
    if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) {
      int one = 1;
      ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      return fd;
    }
    ::close(fd);
    ::usleep(50 * 1000);
  } while (NowMs() < deadline);
  return -1;
}

std::vector<std::pair<int, int>> SplitLayers(int num_layers, int world_size) {
  std::vector<std::pair<int, int>> out;
  const int q = num_layers / world_size, r = num_layers % world_size;
  int lo = 0;
  for (int i = 0; i < world_size; ++i) {
    const int n = q + (i < r ? 1 : 0);
    out.emplace_back(lo, lo + n - 1);
    lo += n;
  }
  return out;
}

// ------------------------------------------------------------------------------------ master
ControlMaster::ControlMaster(const std::string& host, int port, int world_size, int hb_interval_ms, int hb_timeout_ms)
    : world_size_(world_size), hb_interval_ms_(hb_interval_ms), hb_timeout_ms_(hb_timeout_ms) {
  listen_fd_ = ListenOn(host, port, &port_);
  if (listen_fd_ < 0) { alive_ = false; return; }
  accept_thread_ = std::thread(&ControlMaster::AcceptLoop, this);
  hb_thread_ = std::thread(&ControlMaster::HeartbeatLoop, this);
}

ControlMaster::~ControlMaster() { Stop(); }

void ControlMaster::Stop() {
  if (stop_.exchange(true)) return;
  if (listen_fd_ >= 0) { ::shutdown(listen_fd_, SHUT_RDWR); ::close(listen_fd_); }
  cv_.notify_all();
  if (accept_thread_.joinable()) accept_thread_.join();
  if (hb_thread_.joinable()) hb_thread_.join();
  std::vector<Peer*> peers;
  {
    std::lock_guard<std::mutex> g(mu_);
    peers = peers_;
  }
  for (Peer* p : peers) {
    if (p->fd >= 0) ::shutdown(p->fd, SHUT_RDWR);
    if (p->reader.joinable()) p->reader.join();
    if (p->fd >= 0) ::close(p->fd);
    delete p;
  }
  std::lock_guard<std::mutex> g(mu_);
  peers_.clear();
}

void ControlMaster::AcceptLoop() {
  while (!stop_) {
    struct pollfd pfd{listen_fd_, POLLIN, 0};
    if (::poll(&pfd, 1, 200) <= 0) continue;
    const int fd = ::accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) continue;
    int one = 1;
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    Packet hello;
    if (!RecvPacket(fd, &hello, 5000) || hello.type != PKT_ADD_NODE) { ::close(fd); continue; }
    Peer* p = new Peer();
    p->fd = fd;
    p->rank = hello.node_rank;
    p->last_seen_ms = NowMs();
    {
      std::lock_guard<std::mutex> g(mu_);
      peers_.push_back(p);
    }
    Packet ack;
    ack.type = PKT_ADD_NODE_ACK;
    SendPacket(fd, ack);
    p->reader = std::thread(&ControlMaster::ReaderLoop, this, p);
    cv_.notify_all();
  }
}

void ControlMaster::MarkFailed(Peer* p) {
  std::lock_guard<std::mutex> g(mu_);
  if (!p->failed) {
    p->failed = true;
    alive_ = false;   // one lost node stops the cluster (no elastic re-sharding)
    KLLM_LOG_ERROR << "control channel: connection to node " << p->rank << " closed; the cluster is no longer alive";
  }
  cv_.notify_all();
}

void ControlMaster::ReaderLoop(Peer* p) {
  while (!stop_) {
    Packet pkt;
    if (!RecvPacket(p->fd, &pkt, -1)) {
      if (!stop_) MarkFailed(p);
      return;
    }
    std::lock_guard<std::mutex> g(mu_);
    p->last_seen_ms = NowMs();
    if (pkt.type == PKT_HEARTBEAT_REQ) {
      Packet rsp;
      rsp.type = PKT_HEARTBEAT_RSP;
      SendPacket(p->fd, rsp);
    } else {
      pending_[pkt.type][p->rank] = pkt.payload;
      cv_.notify_all();
    }
  }
}

void ControlMaster::HeartbeatLoop() {
  while (!stop_) {
    for (int i = 0; i < hb_interval_ms_ / 20 + 1 && !stop_; ++i) ::usleep(20 * 1000);
    std::lock_guard<std::mutex> g(mu_);
    const int64_t now = NowMs();
    for (Peer* p : peers_) {
      if (!p->failed && now - p->last_seen_ms > hb_timeout_ms_) {
        p->failed = true;
        alive_ = false;
        KLLM_LOG_ERROR << "control channel: no heartbeat from node " << p->rank << " for " << (now - p->last_seen_ms)
                       << " ms; the cluster is no longer alive";
        cv_.notify_all();
      }
    }
  }
}

bool ControlMaster::WaitForNodes(int timeout_ms) {
  std::unique_lock<std::mutex> lk(mu_);
  return cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms),
                      [this] { return static_cast<int>(peers_.size()) >= world_size_ - 1 || stop_; }) && !stop_;
}

bool ControlMaster::Collect(uint16_t type, int timeout_ms, std::map<int, std::string>* values) {
  std::unique_lock<std::mutex> lk(mu_);
  const bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] {
    return static_cast<int>(pending_[type].size()) >= world_size_ - 1 || !alive_ || stop_;
  });
  if (!ok || !alive_ || stop_) return false;
  *values = pending_[type];
  pending_[type].clear();
  return true;
}

void ControlMaster::Reply(uint16_t type, const std::map<int, std::string>& per_rank, const std::string& common) {
  std::lock_guard<std::mutex> g(mu_);
  for (Peer* p : peers_) {
    if (p->failed) continue;
    Packet rsp;
    rsp.type = type;
    auto it = per_rank.find(p->rank);
    rsp.payload = it != per_rank.end() ? it->second : common;
    SendPacket(p->fd, rsp);
  }
}

bool ControlMaster::Barrier(int timeout_ms) {
  std::map<int, std::string> v;
  if (!Collect(PKT_BARRIER_REQ, timeout_ms, &v)) return false;
  Reply(PKT_BARRIER_RSP, {}, "");
  return true;
}

std::vector<std::pair<int, int>> ControlMaster::AssignLayers(int num_layers, int timeout_ms) {
  std::map<int, std::string> v;
  if (!Collect(PKT_LAYER_REQ, timeout_ms, &v)) return {};
  auto ranges = SplitLayers(num_layers, world_size_);
  std::map<int, std::string> per_rank;
  for (int r = 1; r < world_size_; ++r) per_rank[r] = EncodeInts({ranges[r].first, ranges[r].second});
  Reply(PKT_LAYER_RSP, per_rank, "");
  return ranges;
}

int ControlMaster::SyncBlockNum(int my_blocks, int timeout_ms) {
  std::map<int, std::string> v;
  if (!Collect(PKT_BLOCKNUM_REQ, timeout_ms, &v)) return -1;
  int m = my_blocks;
  for (auto& kv : v) {
    auto ints = DecodeInts(kv.second);
    if (!ints.empty()) m = std::min(m, ints[0]);
  }
  Reply(PKT_BLOCKNUM_RSP, {}, EncodeInts({m}));
  return m;
}

bool ControlMaster::Broadcast(const std::string& bytes) {
  if (!alive_) return false;
  Reply(PKT_SCHEDULE, {}, bytes);
  return true;
}

void ControlMaster::ShutdownCluster() { Reply(PKT_SHUTDOWN, {}, ""); }

std::vector<int> ControlMaster::FailedNodes() {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<int> out;
  for (Peer* p : peers_) if (p->failed) out.push_back(p->rank);
  return out;
}

// ------------------------------------------------------------------------------------ worker
ControlWorker::ControlWorker(const std::string& master_host, int master_port, int node_rank, int hb_interval_ms,
                             int hb_timeout_ms)
    : host_(master_host), port_(master_port), rank_(node_rank), hb_interval_ms_(hb_interval_ms),
      hb_timeout_ms_(hb_timeout_ms) {}

ControlWorker::~ControlWorker() { Stop(); }

void ControlWorker::Stop() {
  if (stop_.exchange(true)) return;
  if (fd_ >= 0) ::shutdown(fd_, SHUT_RDWR);
  cv_.notify_all();
  if (reader_.joinable()) reader_.join();
  if (hb_thread_.joinable()) hb_thread_.join();
  if (fd_ >= 0) ::close(fd_);
  fd_ = -1;
}

bool ControlWorker::Connect(int retry_ms) {
  fd_ = ConnectTo(host_, port_, retry_ms);
  if (fd_ < 0) return false;
  Packet hello;
  hello.type = PKT_ADD_NODE;
  hello.node_rank = rank_;
  Packet ack;
  if (!SendPacket(fd_, hello) || !RecvPacket(fd_, &ack, 5000) || ack.type != PKT_ADD_NODE_ACK) return false;
  alive_ = true;
  last_seen_ms_ = NowMs();
  reader_ = std::thread(&ControlWorker::ReaderLoop, this);
  hb_thread_ = std::thread(&ControlWorker::HeartbeatLoop, this);
  return true;
}

void ControlWorker::ReaderLoop() {
  while (!stop_) {
    Packet pkt;
    if (!RecvPacket(fd_, &pkt, -1)) {
      alive_ = false;   // EOF: the master is gone
      if (!stop_) KLLM_LOG_ERROR << "control channel: the master closed the connection";
      cv_.notify_all();
      return;
    }
    last_seen_ms_ = NowMs();
    if (pkt.type == PKT_HEARTBEAT_RSP) continue;
    if (pkt.type == PKT_SHUTDOWN) { shutdown_ = true; alive_ = false; cv_.notify_all(); continue; }
    std::lock_guard<std::mutex> g(mu_);
    inbox_[pkt.type].push_back(std::move(pkt.payload));
    cv_.notify_all();
  }
}

void ControlWorker::HeartbeatLoop() {
  while (!stop_) {
    for (int i = 0; i < hb_interval_ms_ / 20 + 1 && !stop_; ++i) ::usleep(20 * 1000);
    if (stop_ || !alive_) continue;
    Packet hb;
    hb.type = PKT_HEARTBEAT_REQ;
    hb.node_rank = rank_;
    {
      std::lock_guard<std::mutex> g(send_mu_);
      if (!SendPacket(fd_, hb)) { alive_ = false; cv_.notify_all(); }
    }
    if (NowMs() - last_seen_ms_ > hb_timeout_ms_) { alive_ = false; cv_.notify_all(); }
  }
}

bool ControlWorker::Request(uint16_t req, uint16_t rsp, const std::string& payload, std::string* out, int timeout_ms) {
  if (!alive_) return false;
  Packet p;
  p.type = req;
  p.node_rank = rank_;
  p.payload = payload;
  {
    std::lock_guard<std::mutex> g(send_mu_);
    if (!SendPacket(fd_, p)) return false;
  }
  std::unique_lock<std::mutex> lk(mu_);
  const bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms),
                               [&] { return !inbox_[rsp].empty() || !alive_ || stop_; });
  if (!ok || inbox_[rsp].empty()) return false;
  if (out) *out = inbox_[rsp].front();
  inbox_[rsp].pop_front();
  return true;
}

bool ControlWorker::Barrier(int timeout_ms) { return Request(PKT_BARRIER_REQ, PKT_BARRIER_RSP, "", nullptr, timeout_ms); }

std::pair<int, int> ControlWorker::GetLayers(int timeout_ms) {
  std::string out;
  if (!Request(PKT_LAYER_REQ, PKT_LAYER_RSP, "", &out, timeout_ms)) return {-1, -1};
  auto v = DecodeInts(out);
  return v.size() >= 2 ? std::make_pair(v[0], v[1]) : std::make_pair(-1, -1);
}

int ControlWorker::SyncBlockNum(int my_blocks, int timeout_ms) {
  std::string out;
  if (!Request(PKT_BLOCKNUM_REQ, PKT_BLOCKNUM_RSP, EncodeInts({my_blocks}), &out, timeout_ms)) return -1;
  auto v = DecodeInts(out);
  return v.empty() ? -1 : v[0];
}

bool ControlWorker::RecvBroadcast(std::string* bytes, int timeout_ms) {
  std::unique_lock<std::mutex> lk(mu_);
  const bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms),
                               [&] { return !inbox_[PKT_SCHEDULE].empty() || !alive_ || stop_; });
  if (!ok || inbox_[PKT_SCHEDULE].empty()) return false;
  *bytes = std::move(inbox_[PKT_SCHEDULE].front());
  inbox_[PKT_SCHEDULE].pop_front();
  return true;
}

#ifndef KSANA_NO_PYBIND
void BindControlChannel(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("split_layers", &SplitLayers);
  py::class_<ControlMaster>(m, "ControlMaster")
      .def(py::init<const std::string&, int, int, int, int>(), py::arg("host"), py::arg("port"), py::arg("world_size"),
           py::arg("heartbeat_interval_ms") = 30000, py::arg("heartbeat_timeout_ms") = 120000)
      .def_property_readonly("port", &ControlMaster::port)
      .def("wait_for_nodes", &ControlMaster::WaitForNodes, py::call_guard<py::gil_scoped_release>())
      .def("barrier", &ControlMaster::Barrier, py::call_guard<py::gil_scoped_release>())
      .def("assign_layers", &ControlMaster::AssignLayers, py::call_guard<py::gil_scoped_release>())
      .def("sync_block_num", &ControlMaster::SyncBlockNum, py::call_guard<py::gil_scoped_release>())
      .def("broadcast", [](ControlMaster& c, py::bytes b) { return c.Broadcast(std::string(b)); })
      .def("shutdown_cluster", &ControlMaster::ShutdownCluster)
      .def("alive", &ControlMaster::alive)
      .def("failed_nodes", &ControlMaster::FailedNodes)
      .def("stop", &ControlMaster::Stop, py::call_guard<py::gil_scoped_release>());
  py::class_<ControlWorker>(m, "ControlWorker")
      .def(py::init<const std::string&, int, int, int, int>(), py::arg("master_host"), py::arg("master_port"),
           py::arg("node_rank"), py::arg("heartbeat_interval_ms") = 30000, py::arg("heartbeat_timeout_ms") = 120000)
      .def("connect", &ControlWorker::Connect, py::call_guard<py::gil_scoped_release>())
      .def("barrier", &ControlWorker::Barrier, py::call_guard<py::gil_scoped_release>())
      .def("get_layers", &ControlWorker::GetLayers, py::call_guard<py::gil_scoped_release>())
      .def("sync_block_num", &ControlWorker::SyncBlockNum, py::call_guard<py::gil_scoped_release>())
      .def("recv_broadcast", [](ControlWorker& c, int timeout_ms) -> py::object {
        std::string out;
        bool ok;
        {
          py::gil_scoped_release rel;
          ok = c.RecvBroadcast(&out, timeout_ms);
        }
        if (!ok) return py::none();
        return py::bytes(out);
      })
      .def("alive", &ControlWorker::alive)
      .def("shutdown_requested", &ControlWorker::shutdown_requested)
      .def("stop", &ControlWorker::Stop, py::call_guard<py::gil_scoped_release>());
}

#endif  // KSANA_NO_PYBIND

}  // namespace ksana
