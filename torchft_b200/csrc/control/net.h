// Sockets, framed RPC transport, backoff and timeout helpers for the control plane.
//
// One TCP port serves two protocols, told apart by the first bytes of a connection:
//   * framed RPC: every request is  "TFT1" | u32 len | u16 path_len | path |
//     u8 tmo_len | grpc-timeout text | protobuf payload;  every response is
//     u32 len | u8 status code | u16 msg_len | msg | protobuf payload.  Method paths
//     ("/torchft.ManagerService/Quorum") and status codes are those of gRPC.
//   * HTTP/1.1 for the dashboard.
//   * gRPC over HTTP/2 (connections that open with the HTTP/2 client preface), see h2.h: the
//     reference's own wire format.  Servers always accept it; clients use it when the process
//     selects it (set_rpc_protocol("grpc") or TORCHFT_B200_RPC=grpc).
#pragma once

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace tft {
namespace net {

using Clock = std::chrono::steady_clock;
using Millis = std::chrono::milliseconds;

enum Code : int {
  kOk = 0,
  kCancelled = 1,
  kUnknown = 2,
  kInvalidArgument = 3,
  kDeadlineExceeded = 4,
  kNotFound = 5,
  kInternal = 13,
  kUnavailable = 14,
};

const char* code_name(int code);

struct Status {
  int code = kOk;
  std::string message;
  bool ok() const { return code == kOk; }
  static Status Ok() { return {}; }
  static Status Error(int c, std::string m) { return Status{c, std::move(m)}; }
  // "status: Cancelled, message: \"...\"" -- the text Python callers see.
  std::string to_string() const;
};

struct RpcError : std::runtime_error {
  int code;
  RpcError(int c, const std::string& m) : std::runtime_error(Status{c, m}.to_string()), code(c) {}
  bool is_timeout() const { return code == kCancelled || code == kDeadlineExceeded; }
};

// ---- timeouts in grpc-timeout header syntax ("100m", "5S", ...; at most 8 digits)
std::optional<std::chrono::nanoseconds> parse_grpc_timeout(const std::string& text);
std::string format_grpc_timeout(Millis timeout);

// ---- exponential backoff
struct BackoffOptions {
  Millis initial{100};
  Millis max_backoff{10000};
  double factor = 1.5;
  Millis max_jitter{100};
  std::optional<Millis> timeout;      // overall deadline
  std::optional<int> max_retries;
};
// Calls fn until it returns true.  Returns false when retries or time ran out.
bool retry_backoff(const BackoffOptions& opt, const std::function<bool(int attempt)>& fn,
                   int* attempts_out = nullptr);

// ---- addresses
struct HostPort {
  std::string host;
  int port = 0;
};
// Accepts "http://host:port", "host:port", "[v6]:port".
HostPort parse_address(const std::string& addr);
// hostname if it resolves, otherwise "127.0.0.1".
std::string advertised_host(const std::string& hostname);
std::string local_hostname();

int listen_on(const std::string& bind, int* port_out);                 // throws std::runtime_error
int connect_to(const HostPort& hp, Millis timeout, std::string* err);  // -1 on failure

// ---- blocking I/O with a deadline (poll based; `stopping` aborts a read early)
enum IoResult { kIoOk, kIoTimeout, kIoClosed };
IoResult read_exact(int fd, char* buf, size_t n, Clock::time_point deadline, const std::atomic<bool>* stopping);
IoResult write_all(int fd, const char* buf, size_t n, Clock::time_point deadline);

// ---- wire protocol used by Client objects of this process: "framed" (default) or "grpc"
void set_rpc_protocol(const std::string& name);  // throws std::invalid_argument
std::string rpc_protocol();

// ---- server
struct CallContext {
  std::optional<std::chrono::nanoseconds> timeout;  // from the request header
  Clock::time_point deadline = Clock::time_point::max();
  int fd = -1;  // framed transport: the connection (one call at a time); -1 on multiplexed transports
  const std::atomic<bool>* stopping = nullptr;
  const std::atomic<bool>* stream_cancelled = nullptr;  // HTTP/2: set when the peer reset the stream or went away
  // True once the deadline passed, the peer hung up or the server is shutting down.
  bool cancelled() const;
};

struct HttpRequest {
  std::string method, path, body;
};
struct HttpResponse {
  int status = 200;
  std::string content_type = "text/html; charset=utf-8";
  std::string body;
};

class Server {
 public:
  using Handler = std::function<Status(const CallContext&, const std::string&, std::string*)>;
  using HttpHandler = std::function<HttpResponse(const HttpRequest&)>;

  explicit Server(const std::string& bind);
  ~Server();
  void add_method(const std::string& path, Handler h) { methods_[path] = std::move(h); }
  void set_http_handler(HttpHandler h) { http_ = std::move(h); }
  void start();
  void shutdown();
  int port() const { return port_; }
  const std::atomic<bool>& stopping() const { return stopping_; }

 private:
  void accept_loop();
  void serve(int fd);
  void serve_rpc(int fd);
  void serve_http(int fd, const std::string& first);

  int listen_fd_ = -1;
  int port_ = 0;
  std::map<std::string, Handler> methods_;
  HttpHandler http_;
  std::thread accept_thread_;
  std::atomic<bool> stopping_{false};
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<int> conn_fds_;
  int active_ = 0;
};

// ---- client
class Client {
 public:
  // Connects with exponential backoff until connect_timeout; throws RpcError(kUnavailable).
  Client(const std::string& addr, Millis connect_timeout);
  ~Client();
  // Throws RpcError.  A client-side timeout raises kCancelled "Timeout expired".
  std::string call(const std::string& path, const std::string& payload,
                   std::optional<Millis> timeout);
  const std::string& address() const { return addr_; }

 private:
  void ensure_connected();
  void close_fd();
  std::string call_grpc(const std::string& path, const std::string& payload, std::optional<Millis> timeout);
  std::string addr_;
  HostPort hp_;
  Millis connect_timeout_;
  std::mutex mu_;
  int fd_ = -1;
  bool grpc_ = false;                          // fixed at construction from rpc_protocol()
  std::shared_ptr<void> h2_;                   // h2::ClientConnection, owns the socket in gRPC mode
};

void log_info(const std::string& module, const std::string& msg);
// Per-request chatter; printed only when TORCHFT_B200_LOG=debug.
void log_debug(const std::string& module, const std::string& msg);
void set_log_enabled(bool enabled);

}  // namespace net
}  // namespace tft
