#include "net.h"

#include "h2.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <signal.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <random>
#include <sstream>

namespace tft {
namespace net {

namespace {

std::atomic<bool> g_log_enabled{true};

void put_u32(std::string* s, uint32_t v) {
  char b[4] = {char(v >> 24), char(v >> 16), char(v >> 8), char(v)};
  s->append(b, 4);
}
void put_u16(std::string* s, uint16_t v) {
  char b[2] = {char(v >> 8), char(v)};
  s->append(b, 2);
}
uint32_t get_u32(const char* p) {
  const unsigned char* u = reinterpret_cast<const unsigned char*>(p);
  return (uint32_t(u[0]) << 24) | (uint32_t(u[1]) << 16) | (uint32_t(u[2]) << 8) | uint32_t(u[3]);
}
uint16_t get_u16(const char* p) {
  const unsigned char* u = reinterpret_cast<const unsigned char*>(p);
  return uint16_t((u[0] << 8) | u[1]);
}

int remaining_ms(Clock::time_point deadline) {
  if (deadline == Clock::time_point::max()) return 200;
  auto left = std::chrono::duration_cast<Millis>(deadline - Clock::now()).count();
  if (left <= 0) return 0;
  return static_cast<int>(std::min<long long>(left, 200));
}

}  // namespace

IoResult read_exact(int fd, char* buf, size_t n, Clock::time_point deadline,
                    const std::atomic<bool>* stopping) {
  size_t got = 0;
  while (got < n) {
    if (stopping && stopping->load()) return kIoClosed;
    if (deadline != Clock::time_point::max() && Clock::now() >= deadline) return kIoTimeout;
    struct pollfd p = {fd, POLLIN, 0};
    int pr = ::poll(&p, 1, remaining_ms(deadline));
    if (pr < 0) {
      if (errno == EINTR) continue;
      return kIoClosed;
    }
    if (pr == 0) continue;
    ssize_t r = ::recv(fd, buf + got, n - got, 0);
    if (r == 0) return kIoClosed;
    if (r < 0) {
      if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
      return kIoClosed;
    }
    got += static_cast<size_t>(r);
  }
  return kIoOk;
}

IoResult write_all(int fd, const char* buf, size_t n, Clock::time_point deadline) {
  size_t sent = 0;
  while (sent < n) {
    if (deadline != Clock::time_point::max() && Clock::now() >= deadline) return kIoTimeout;
    struct pollfd p = {fd, POLLOUT, 0};
    int pr = ::poll(&p, 1, remaining_ms(deadline));
    if (pr < 0) {
      if (errno == EINTR) continue;
      return kIoClosed;
    }
    if (pr == 0) continue;
    ssize_t r = ::send(fd, buf + sent, n - sent, MSG_NOSIGNAL);
    if (r < 0) {
      if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
      return kIoClosed;
    }
    sent += static_cast<size_t>(r);
  }
  return kIoOk;
}

namespace {

std::atomic<int> g_rpc_protocol{-1};  // -1: not decided yet (environment), 0 framed, 1 grpc

void set_nodelay(int fd) {
  int one = 1;
  ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  ::setsockopt(fd, SOL_SOCKET, SO_KEEPALIVE, &one, sizeof(one));
}

}  // namespace

void set_log_enabled(bool enabled) { g_log_enabled.store(enabled); }

void set_rpc_protocol(const std::string& name) {
  if (name == "framed") g_rpc_protocol.store(0);
  else if (name == "grpc") g_rpc_protocol.store(1);
  else throw std::invalid_argument("unknown RPC protocol '" + name + "' (framed or grpc)");
}

std::string rpc_protocol() {
  int v = g_rpc_protocol.load();
  if (v < 0) {
    const char* env = std::getenv("TORCHFT_B200_RPC");
    v = (env != nullptr && std::string(env) == "grpc") ? 1 : 0;
    g_rpc_protocol.store(v);
  }
  return v == 1 ? "grpc" : "framed";
}

void log_info(const std::string& module, const std::string& msg) {
  if (!g_log_enabled.load()) return;
  struct timeval tv;
  gettimeofday(&tv, nullptr);
  struct tm tmv;
  time_t secs = tv.tv_sec;
  gmtime_r(&secs, &tmv);
  char ts[64];
  strftime(ts, sizeof(ts), "%Y-%m-%dT%H:%M:%S", &tmv);
  char line[128];
  snprintf(line, sizeof(line), "%s.%03d", ts, static_cast<int>(tv.tv_usec / 1000));
  // colour only when asked for (CLICOLOR_FORCE, as the reference's logger) and never into a pipe by default
  static const bool colour = [] {
    const char* v = std::getenv("CLICOLOR_FORCE");
    return v != nullptr && std::string(v) != "0" && std::string(v) != "";
  }();
  const std::string level = colour ? "\x1b[32mINFO\x1b[0m" : "INFO";
  std::string out = std::string(line) + " - " + level + " - [" + module + "] " + msg + "\n";
  ssize_t ignored = ::write(2, out.data(), out.size());
  (void)ignored;
}

void log_debug(const std::string& module, const std::string& msg) {
  static const bool enabled = [] {
    const char* v = std::getenv("TORCHFT_B200_LOG");
    return v && std::string(v) == "debug";
  }();
  if (enabled) log_info(module, msg);
}

const char* code_name(int code) {
  switch (code) {
    case kOk: return "Ok";
    case kCancelled: return "Cancelled";
    case kUnknown: return "Unknown";
    case kInvalidArgument: return "InvalidArgument";
    case kDeadlineExceeded: return "DeadlineExceeded";
    case kNotFound: return "NotFound";
    case kInternal: return "Internal";
    case kUnavailable: return "Unavailable";
    default: return "Unknown";
  }
}

std::string Status::to_string() const {
  return std::string("status: ") + code_name(code) + ", message: \"" + message + "\"";
}

std::optional<std::chrono::nanoseconds> parse_grpc_timeout(const std::string& text) {
  if (text.size() < 2 || text.size() > 9) return std::nullopt;
  const char unit = text.back();
  uint64_t value = 0;
  for (size_t i = 0; i + 1 < text.size(); ++i) {
    if (text[i] < '0' || text[i] > '9') return std::nullopt;
    value = value * 10 + static_cast<uint64_t>(text[i] - '0');
  }
  using namespace std::chrono;
  switch (unit) {
    case 'H': return duration_cast<nanoseconds>(hours(value));
    case 'M': return duration_cast<nanoseconds>(minutes(value));
    case 'S': return duration_cast<nanoseconds>(seconds(value));
    case 'm': return duration_cast<nanoseconds>(milliseconds(value));
    case 'u': return duration_cast<nanoseconds>(microseconds(value));
    case 'n': return nanoseconds(value);
    default: return std::nullopt;
  }
}

std::string format_grpc_timeout(Millis timeout) {
  long long ms = std::max<long long>(timeout.count(), 0);
  if (ms <= 99999999LL) return std::to_string(ms) + "m";
  long long s = ms / 1000;
  if (s <= 99999999LL) return std::to_string(s) + "S";
  return std::to_string(std::min<long long>(s / 60, 99999999LL)) + "M";
}

bool retry_backoff(const BackoffOptions& opt, const std::function<bool(int)>& fn, int* attempts_out) {
  static thread_local std::mt19937_64 rng{std::random_device{}()};
  const auto start = Clock::now();
  Millis backoff = opt.initial;
  int attempt = 0;
  while (true) {
    if (fn(attempt)) {
      if (attempts_out) *attempts_out = attempt + 1;
      return true;
    }
    ++attempt;
    if (attempts_out) *attempts_out = attempt;
    if (opt.max_retries && attempt > *opt.max_retries) return false;
    Millis jitter{0};
    if (opt.max_jitter.count() > 0)
      jitter = Millis(static_cast<long long>(rng() % static_cast<uint64_t>(opt.max_jitter.count() + 1)));
    Millis sleep_for = backoff + jitter;
    if (opt.timeout) {
      auto elapsed = std::chrono::duration_cast<Millis>(Clock::now() - start);
      if (elapsed >= *opt.timeout) return false;
      sleep_for = std::min(sleep_for, *opt.timeout - elapsed);
    }
    std::this_thread::sleep_for(sleep_for);
    backoff = std::min(Millis(static_cast<long long>(backoff.count() * opt.factor)), opt.max_backoff);
  }
}

HostPort parse_address(const std::string& addr_in) {
  std::string a = addr_in;
  auto scheme = a.find("://");
  if (scheme != std::string::npos) a = a.substr(scheme + 3);
  auto slash = a.find('/');
  if (slash != std::string::npos) a = a.substr(0, slash);
  HostPort hp;
  if (!a.empty() && a[0] == '[') {
    auto close = a.find(']');
    if (close == std::string::npos) throw std::runtime_error("invalid address: " + addr_in);
    hp.host = a.substr(1, close - 1);
    if (close + 2 <= a.size() && a[close + 1] == ':') hp.port = std::atoi(a.c_str() + close + 2);
  } else {
    auto colon = a.rfind(':');
    if (colon == std::string::npos) throw std::runtime_error("address has no port: " + addr_in);
    hp.host = a.substr(0, colon);
    hp.port = std::atoi(a.c_str() + colon + 1);
  }
  if (hp.host.empty()) hp.host = "127.0.0.1";
  return hp;
}

std::string local_hostname() {
  char buf[256];
  if (::gethostname(buf, sizeof(buf)) != 0) return "localhost";
  buf[sizeof(buf) - 1] = 0;
  return buf;
}

std::string advertised_host(const std::string& hostname) {
  struct addrinfo hints;
  std::memset(&hints, 0, sizeof(hints));
  hints.ai_socktype = SOCK_STREAM;
  struct addrinfo* res = nullptr;
  if (!hostname.empty() && ::getaddrinfo(hostname.c_str(), nullptr, &hints, &res) == 0 && res) {
    ::freeaddrinfo(res);
    return hostname;
  }
  return "127.0.0.1";
}

int listen_on(const std::string& bind, int* port_out) {
  HostPort hp;
  if (!bind.empty() && bind[0] == ':') hp = HostPort{"::", std::atoi(bind.c_str() + 1)};
  else hp = parse_address(bind);
  int fd = -1;
  bool v6 = hp.host.find(':') != std::string::npos;
  if (v6) {
    fd = ::socket(AF_INET6, SOCK_STREAM, 0);
    if (fd >= 0) {
      int zero = 0, one = 1;
      ::setsockopt(fd, IPPROTO_IPV6, IPV6_V6ONLY, &zero, sizeof(zero));
      ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
      struct sockaddr_in6 sa;
      std::memset(&sa, 0, sizeof(sa));
      sa.sin6_family = AF_INET6;
      sa.sin6_port = htons(static_cast<uint16_t>(hp.port));
      if (::inet_pton(AF_INET6, hp.host.c_str(), &sa.sin6_addr) != 1) sa.sin6_addr = in6addr_any;
      if (::bind(fd, reinterpret_cast<struct sockaddr*>(&sa), sizeof(sa)) != 0) {
        ::close(fd);
        fd = -1;
      }
    }
    if (fd < 0) {  // no IPv6 on this host: fall back to the IPv4 wildcard
      hp.host = "0.0.0.0";
      v6 = false;
    }
  }
  if (!v6) {
    fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) throw std::runtime_error(std::string("socket: ") + strerror(errno));
    int one = 1;
    ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    struct sockaddr_in sa;
    std::memset(&sa, 0, sizeof(sa));
    sa.sin_family = AF_INET;
    sa.sin_port = htons(static_cast<uint16_t>(hp.port));
    if (hp.host == "localhost") hp.host = "127.0.0.1";
    if (::inet_pton(AF_INET, hp.host.c_str(), &sa.sin_addr) != 1) sa.sin_addr.s_addr = INADDR_ANY;
    if (::bind(fd, reinterpret_cast<struct sockaddr*>(&sa), sizeof(sa)) != 0) {
      std::string e = strerror(errno);
      ::close(fd);
      throw std::runtime_error("bind " + bind + ": " + e);
    }
  }
  if (::listen(fd, 1024) != 0) {
    std::string e = strerror(errno);
    ::close(fd);
    throw std::runtime_error("listen: " + e);
  }
  struct sockaddr_storage ss;
  socklen_t len = sizeof(ss);
  ::getsockname(fd, reinterpret_cast<struct sockaddr*>(&ss), &len);
  int port = ss.ss_family == AF_INET6 ? ntohs(reinterpret_cast<struct sockaddr_in6*>(&ss)->sin6_port)
                                      : ntohs(reinterpret_cast<struct sockaddr_in*>(&ss)->sin_port);
  if (port_out) *port_out = port;
  return fd;
}

int connect_to(const HostPort& hp, Millis timeout, std::string* err) {
  struct addrinfo hints;
  std::memset(&hints, 0, sizeof(hints));
  hints.ai_socktype = SOCK_STREAM;
  hints.ai_family = AF_UNSPEC;
  struct addrinfo* res = nullptr;
  std::string port = std::to_string(hp.port);
  int gai = ::getaddrinfo(hp.host.c_str(), port.c_str(), &hints, &res);
  if (gai != 0 || !res) {
    if (err) *err = std::string("resolve ") + hp.host + ": " + gai_strerror(gai);
    return -1;
  }
  int fd = -1;
  std::string last = "no addresses";
  for (struct addrinfo* ai = res; ai; ai = ai->ai_next) {
    fd = ::socket(ai->ai_family, ai->ai_socktype, ai->ai_protocol);
    if (fd < 0) continue;
    int flags = ::fcntl(fd, F_GETFL, 0);
    ::fcntl(fd, F_SETFL, flags | O_NONBLOCK);
    int rc = ::connect(fd, ai->ai_addr, ai->ai_addrlen);
    if (rc != 0 && errno == EINPROGRESS) {
      struct pollfd p = {fd, POLLOUT, 0};
      int pr = ::poll(&p, 1, static_cast<int>(std::max<long long>(timeout.count(), 1)));
      if (pr > 0) {
        int soerr = 0;
        socklen_t sl = sizeof(soerr);
        ::getsockopt(fd, SOL_SOCKET, SO_ERROR, &soerr, &sl);
        rc = soerr == 0 ? 0 : -1;
        if (soerr) last = strerror(soerr);
      } else {
        rc = -1;
        last = "connect timed out";
      }
    } else if (rc != 0) {
      last = strerror(errno);
    }
    if (rc == 0) {
      set_nodelay(fd);
      break;
    }
    ::close(fd);
    fd = -1;
  }
  ::freeaddrinfo(res);
  if (fd < 0 && err) *err = "connect " + hp.host + ":" + port + ": " + last;
  return fd;
}

bool CallContext::cancelled() const {
  if (stopping && stopping->load()) return true;
  if (stream_cancelled && stream_cancelled->load()) return true;
  if (deadline != Clock::time_point::max() && Clock::now() >= deadline) return true;
  if (fd >= 0) {
    char c;
    ssize_t r = ::recv(fd, &c, 1, MSG_PEEK | MSG_DONTWAIT);
    if (r == 0) return true;
    if (r < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return true;
  }
  return false;
}

// ---------------------------------------------------------------- Server
Server::Server(const std::string& bind) { listen_fd_ = listen_on(bind, &port_); }

Server::~Server() { shutdown(); }

void Server::start() { accept_thread_ = std::thread([this] { accept_loop(); }); }

void Server::shutdown() {
  bool was = stopping_.exchange(true);
  if (was) {
    if (accept_thread_.joinable()) accept_thread_.join();
    return;
  }
  if (listen_fd_ >= 0) ::shutdown(listen_fd_, SHUT_RDWR);
  if (accept_thread_.joinable()) accept_thread_.join();
  if (listen_fd_ >= 0) {
    ::close(listen_fd_);
    listen_fd_ = -1;
  }
  std::unique_lock<std::mutex> lk(mu_);
  for (int fd : conn_fds_) ::shutdown(fd, SHUT_RDWR);
  cv_.wait_for(lk, std::chrono::seconds(5), [this] { return active_ == 0; });
}

void Server::accept_loop() {
  while (!stopping_.load()) {
    struct pollfd p = {listen_fd_, POLLIN, 0};
    int pr = ::poll(&p, 1, 100);
    if (pr <= 0) continue;
    int fd = ::accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) {
      if (stopping_.load()) break;
      continue;
    }
    set_nodelay(fd);
    {
      std::lock_guard<std::mutex> g(mu_);
      conn_fds_.push_back(fd);
      ++active_;
    }
    std::thread([this, fd] {
      serve(fd);
      ::close(fd);
      std::lock_guard<std::mutex> g(mu_);
      conn_fds_.erase(std::remove(conn_fds_.begin(), conn_fds_.end(), fd), conn_fds_.end());
      --active_;
      cv_.notify_all();
    }).detach();
  }
}

void Server::serve(int fd) {
  char magic[4];
  if (read_exact(fd, magic, 4, Clock::time_point::max(), &stopping_) != kIoOk) return;
  if (std::memcmp(magic, "TFT1", 4) == 0) {
    serve_rpc(fd);
  } else if (std::memcmp(magic, "PRI ", 4) == 0) {
    // HTTP/2 client preface: gRPC
    h2::serve_connection(fd, std::string(magic, 4), stopping_,
                         [this](const std::string& path, const CallContext& ctx, const std::string& payload,
                                std::string* resp) -> Status {
                           auto it = methods_.find(path);
                           if (it == methods_.end()) return Status::Error(12 /*Unimplemented*/, "unknown method " + path);
                           return it->second(ctx, payload, resp);
                         });
  } else {
    serve_http(fd, std::string(magic, 4));
  }
}

void Server::serve_rpc(int fd) {
  bool have_magic = true;
  while (!stopping_.load()) {
    char hdr[4];
    if (!have_magic) {
      if (read_exact(fd, hdr, 4, Clock::time_point::max(), &stopping_) != kIoOk) return;
      if (std::memcmp(hdr, "TFT1", 4) != 0) return;
    }
    have_magic = false;
    if (read_exact(fd, hdr, 4, Clock::time_point::max(), &stopping_) != kIoOk) return;
    uint32_t len = get_u32(hdr);
    if (len < 3 || len > (64u << 20)) return;
    std::string body(len, '\0');
    if (read_exact(fd, &body[0], len, Clock::now() + std::chrono::seconds(30), &stopping_) != kIoOk) return;
    size_t off = 0;
    uint16_t plen = get_u16(body.data());
    off += 2;
    if (off + plen + 1 > body.size()) return;
    std::string path = body.substr(off, plen);
    off += plen;
    uint8_t tlen = static_cast<uint8_t>(body[off++]);
    if (off + tlen > body.size()) return;
    std::string tmo = body.substr(off, tlen);
    off += tlen;
    std::string payload = body.substr(off);

    CallContext ctx;
    ctx.fd = fd;
    ctx.stopping = &stopping_;
    if (!tmo.empty()) {
      ctx.timeout = parse_grpc_timeout(tmo);
      if (ctx.timeout) ctx.deadline = Clock::now() + std::chrono::duration_cast<Clock::duration>(*ctx.timeout);
    }
    Status st;
    std::string resp;
    auto it = methods_.find(path);
    if (it == methods_.end()) {
      st = Status::Error(12 /*Unimplemented*/, "unknown method " + path);
    } else if (!tmo.empty() && !ctx.timeout) {
      st = Status::Error(kInvalidArgument, "invalid timeout " + tmo);
    } else {
      try {
        st = it->second(ctx, payload, &resp);
      } catch (const std::exception& e) {
        st = Status::Error(kInternal, e.what());
      }
    }
    std::string out;
    std::string frame;
    frame.push_back(static_cast<char>(st.code));
    std::string msg = st.message.substr(0, 60000);
    put_u16(&frame, static_cast<uint16_t>(msg.size()));
    frame.append(msg);
    if (st.ok()) frame.append(resp);
    put_u32(&out, static_cast<uint32_t>(frame.size()));
    out.append(frame);
    if (write_all(fd, out.data(), out.size(), Clock::now() + std::chrono::seconds(30)) != kIoOk) return;
  }
}

void Server::serve_http(int fd, const std::string& first) {
  std::string buf = first;
  const auto deadline = Clock::now() + std::chrono::seconds(10);
  size_t header_end;
  while ((header_end = buf.find("\r\n\r\n")) == std::string::npos) {
    char c[1024];
    struct pollfd p = {fd, POLLIN, 0};
    if (Clock::now() >= deadline || stopping_.load()) return;
    if (::poll(&p, 1, 100) <= 0) continue;
    ssize_t r = ::recv(fd, c, sizeof(c), 0);
    if (r <= 0) return;
    buf.append(c, static_cast<size_t>(r));
    if (buf.size() > (1u << 20)) return;
  }
  HttpRequest req;
  {
    std::istringstream is(buf.substr(0, buf.find("\r\n")));
    std::string version;
    is >> req.method >> req.path >> version;
  }
  size_t content_length = 0;
  {
    std::string headers = buf.substr(0, header_end);
    std::string lower = headers;
    std::transform(lower.begin(), lower.end(), lower.begin(), ::tolower);
    auto pos = lower.find("content-length:");
    if (pos != std::string::npos) content_length = static_cast<size_t>(std::atoll(headers.c_str() + pos + 15));
  }
  req.body = buf.substr(header_end + 4);
  if (content_length > (1u << 20)) return;
  if (req.body.size() < content_length) {
    size_t have = req.body.size();
    req.body.resize(content_length);
    if (read_exact(fd, &req.body[have], content_length - have, deadline, &stopping_) != kIoOk) return;
  }
  HttpResponse resp;
  if (http_) {
    try {
      resp = http_(req);
    } catch (const std::exception& e) {
      resp.status = 500;
      resp.content_type = "text/plain";
      resp.body = std::string("Something went wrong: ") + e.what();
    }
  } else {
    resp.status = 404;
    resp.body = "not found";
  }
  const char* reason = resp.status == 200 ? "OK" : resp.status == 404 ? "Not Found"
                     : resp.status == 400 ? "Bad Request" : "Internal Server Error";
  std::string out = "HTTP/1.1 " + std::to_string(resp.status) + " " + reason + "\r\n";
  out += "Content-Type: " + resp.content_type + "\r\n";
  out += "Content-Length: " + std::to_string(resp.body.size()) + "\r\n";
  out += "Connection: close\r\n\r\n";
  out += resp.body;
  write_all(fd, out.data(), out.size(), Clock::now() + std::chrono::seconds(10));
}

// ---------------------------------------------------------------- Client
Client::Client(const std::string& addr, Millis connect_timeout)
    : addr_(addr), hp_(parse_address(addr)), connect_timeout_(connect_timeout) {
  grpc_ = rpc_protocol() == "grpc";
  std::lock_guard<std::mutex> g(mu_);
  ensure_connected();
}

Client::~Client() { close_fd(); }

void Client::close_fd() {
  if (h2_) {  // the HTTP/2 connection owns the socket
    h2_.reset();
    fd_ = -1;
    return;
  }
  if (fd_ >= 0) {
    ::close(fd_);
    fd_ = -1;
  }
}

void Client::ensure_connected() {
  if (fd_ >= 0) return;
  BackoffOptions opt;
  opt.timeout = connect_timeout_;
  std::string err;
  const auto start = Clock::now();
  bool ok = retry_backoff(opt, [&](int) {
    auto elapsed = std::chrono::duration_cast<Millis>(Clock::now() - start);
    Millis left = std::max(connect_timeout_ - elapsed, Millis(1));
    fd_ = connect_to(hp_, left, &err);
    return fd_ >= 0;
  });
  if (!ok) throw RpcError(kUnavailable, "failed to connect to " + addr_ + ": " + err);
  if (grpc_) h2_ = std::make_shared<h2::ClientConnection>(fd_, hp_.host + ":" + std::to_string(hp_.port));
}

std::string Client::call_grpc(const std::string& path, const std::string& payload, std::optional<Millis> timeout) {
  auto* conn = static_cast<h2::ClientConnection*>(h2_.get());
  std::string resp;
  bool broken = false;
  const Status st = conn->call(path, payload, timeout, &resp, &broken);
  if (broken) close_fd();
  if (!st.ok()) throw RpcError(st.code, st.message);
  return resp;
}

std::string Client::call(const std::string& path, const std::string& payload,
                         std::optional<Millis> timeout) {
  std::lock_guard<std::mutex> g(mu_);
  ensure_connected();
  if (grpc_) return call_grpc(path, payload, timeout);
  const auto deadline = timeout ? Clock::now() + *timeout : Clock::time_point::max();
  std::string body;
  put_u16(&body, static_cast<uint16_t>(path.size()));
  body.append(path);
  std::string tmo = timeout ? format_grpc_timeout(*timeout) : std::string();
  body.push_back(static_cast<char>(tmo.size()));
  body.append(tmo);
  body.append(payload);
  std::string out = "TFT1";
  put_u32(&out, static_cast<uint32_t>(body.size()));
  out.append(body);
  IoResult r = write_all(fd_, out.data(), out.size(), deadline);
  if (r != kIoOk) {
    close_fd();
    if (r == kIoTimeout) throw RpcError(kCancelled, "Timeout expired");
    throw RpcError(kUnavailable, "connection to " + addr_ + " lost while sending " + path);
  }
  char hdr[4];
  r = read_exact(fd_, hdr, 4, deadline, nullptr);
  if (r != kIoOk) {
    close_fd();
    if (r == kIoTimeout) throw RpcError(kCancelled, "Timeout expired");
    throw RpcError(kUnavailable, "connection to " + addr_ + " closed during " + path);
  }
  uint32_t len = get_u32(hdr);
  if (len < 3 || len > (64u << 20)) {
    close_fd();
    throw RpcError(kInternal, "malformed response frame");
  }
  std::string frame(len, '\0');
  r = read_exact(fd_, &frame[0], len, deadline, nullptr);
  if (r != kIoOk) {
    close_fd();
    if (r == kIoTimeout) throw RpcError(kCancelled, "Timeout expired");
    throw RpcError(kUnavailable, "connection to " + addr_ + " closed during " + path);
  }
  int code = static_cast<unsigned char>(frame[0]);
  uint16_t mlen = get_u16(frame.data() + 1);
  if (3u + mlen > frame.size()) {
    close_fd();
    throw RpcError(kInternal, "malformed response frame");
  }
  std::string msg = frame.substr(3, mlen);
  if (code != kOk) throw RpcError(code, msg);
  return frame.substr(3 + mlen);
}

}  // namespace net
}  // namespace tft
