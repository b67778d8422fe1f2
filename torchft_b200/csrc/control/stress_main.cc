// Stress harness for the control plane, meant to be built with -fsanitize=thread or
// -fsanitize=address (tests/test_sanitizers.py does both).  One process hosts a lighthouse,
// several replica-group manager servers and one client thread per (group, local rank); the
// threads run quorum + should_commit rounds against each other while another thread polls the
// dashboard.  Half way through one group goes away (its threads stop, its server shuts down),
// so the survivors exercise the heartbeat-expiry and shrinking-quorum paths.  Exit code 0
// means every answer was consistent; the sanitizer reports races and memory errors itself.
//
// The reference relies on Rust's ownership rules for this (src/lighthouse.rs, src/manager.rs);
// a C++ control plane needs a dynamic check instead.
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "h2.h"
#include "lighthouse.h"
#include "manager.h"

using namespace tft;
using net::Millis;

namespace {

std::atomic<int> g_failures{0};

void fail(const std::string& what) {
  std::fprintf(stderr, "stress: %s\n", what.c_str());
  g_failures.fetch_add(1);
}

std::string http_get(int port, const std::string& path) {
  std::string err;
  net::HostPort hp{"127.0.0.1", port};
  const int fd = net::connect_to(hp, Millis(2000), &err);
  if (fd < 0) return "";
  const std::string req = "GET " + path + " HTTP/1.1\r\nHost: x\r\nConnection: close\r\n\r\n";
  std::string out;
  size_t sent = 0;
  while (sent < req.size()) {
    const ssize_t n = ::send(fd, req.data() + sent, req.size() - sent, MSG_NOSIGNAL);
    if (n <= 0) break;
    sent += static_cast<size_t>(n);
  }
  char buf[4096];
  while (sent == req.size()) {
    const ssize_t n = ::recv(fd, buf, sizeof(buf), 0);
    if (n <= 0) break;
    out.append(buf, static_cast<size_t>(n));
  }
  ::close(fd);
  return out;
}

// Connects like an HTTP/2 client and then sends random frames: the server may drop the connection,
// it must not misbehave (the sanitizers watch the parser).
void garbage_client(int port, unsigned seed) {
  std::string err;
  net::HostPort hp{"127.0.0.1", port};
  const int fd = net::connect_to(hp, Millis(2000), &err);
  if (fd < 0) return;
  std::string out = "PRI * HTTP/2.0\r\n\r\nSM\r\n\r\n";
  out += std::string("\0\0\0\4\0\0\0\0\0", 9);  // empty SETTINGS
  unsigned state = seed * 2654435761u + 1;
  auto next = [&state] {
    state = state * 1664525u + 1013904223u;
    return state >> 8;
  };
  const int frames = 1 + static_cast<int>(next() % 40);
  for (int i = 0; i < frames; ++i) {
    const unsigned len = next() % 80;
    const unsigned streams[] = {0, 1, 1, 3, 5, 2, 0x7fffffffu};
    const unsigned stream = streams[next() % 7];
    out.push_back(0);
    out.push_back(0);
    out.push_back(static_cast<char>(len));
    out.push_back(static_cast<char>(next() % 12));
    out.push_back(static_cast<char>(next() & 0xff));
    out.push_back(static_cast<char>((stream >> 24) & 0x7f));
    out.push_back(static_cast<char>((stream >> 16) & 0xff));
    out.push_back(static_cast<char>((stream >> 8) & 0xff));
    out.push_back(static_cast<char>(stream & 0xff));
    for (unsigned j = 0; j < len; ++j) out.push_back(static_cast<char>(next() & 0xff));
  }
  size_t sent = 0;
  while (sent < out.size()) {
    const ssize_t n = ::send(fd, out.data() + sent, out.size() - sent, MSG_NOSIGNAL);
    if (n <= 0) break;
    sent += static_cast<size_t>(n);
  }
  ::shutdown(fd, SHUT_WR);
  char buf[4096];
  while (::recv(fd, buf, sizeof(buf), 0) > 0) {
  }
  ::close(fd);
}

// Feeds random and truncated buffers to every protobuf decoder and to the HPACK decoder; under
// AddressSanitizer an out-of-bounds read in a parser shows up here.
void fuzz_decoders() {
  unsigned state = 12345;
  auto next = [&state] {
    state = state * 1664525u + 1013904223u;
    return state >> 8;
  };
  wire::QuorumMember m;
  m.replica_id = "replica";
  m.address = "http://host:1";
  m.store_address = "host:2";
  m.step = 7;
  m.world_size = 3;
  wire::Quorum q;
  q.quorum_id = 5;
  q.participants = {m, m};
  const std::string good = q.encode();
  for (int i = 0; i < 20000; ++i) {
    std::string buf;
    if (i % 3 == 0) {
      buf = good.substr(0, next() % (good.size() + 1));
      if (!buf.empty()) buf[next() % buf.size()] = static_cast<char>(next() & 0xff);
    } else {
      const unsigned len = next() % 48;
      for (unsigned j = 0; j < len; ++j) buf.push_back(static_cast<char>(next() & 0xff));
    }
    try { wire::QuorumMember::decode(buf); } catch (const std::exception&) {}
    try { wire::Quorum::decode(buf); } catch (const std::exception&) {}
    try { wire::LighthouseQuorumRequest::decode(buf); } catch (const std::exception&) {}
    try { wire::ManagerQuorumRequest::decode(buf); } catch (const std::exception&) {}
    try { wire::ManagerQuorumResponse::decode(buf); } catch (const std::exception&) {}
    try { wire::ShouldCommitRequest::decode(buf); } catch (const std::exception&) {}
    try { wire::KillRequest::decode(buf); } catch (const std::exception&) {}
    std::vector<net::h2::Header> headers;
    net::h2::HpackDecoder().decode(buf, &headers);
    std::string text;
    net::h2::huffman_decode(reinterpret_cast<const uint8_t*>(buf.data()), buf.size(), &text);
  }
}

}  // namespace

int main(int argc, char** argv) {
  const int groups = argc > 1 ? std::atoi(argv[1]) : 3;
  const int ranks = argc > 2 ? std::atoi(argv[2]) : 2;
  const int rounds = argc > 3 ? std::atoi(argv[3]) : 24;
  net::set_log_enabled(false);
  fuzz_decoders();
  if (argc > 4) net::set_rpc_protocol(argv[4]);  // "framed" or "grpc": wire protocol of every client in here

  LighthouseOptions opt;
  opt.bind = "[::]:0";
  opt.min_replicas = 1;
  opt.join_timeout_ms = 200;
  opt.quorum_tick_ms = 5;
  opt.heartbeat_timeout_ms = 300;
  auto lighthouse = std::make_unique<Lighthouse>(opt);
  const std::string lh_addr = "http://127.0.0.1:" + std::to_string(lighthouse->port());

  std::vector<std::unique_ptr<ManagerServer>> managers;
  for (int g = 0; g < groups; ++g)
    managers.push_back(std::make_unique<ManagerServer>("group" + std::to_string(g), lh_addr, "127.0.0.1", "[::]:0",
                                                       "store" + std::to_string(g), static_cast<uint64_t>(ranks),
                                                       Millis(20), Millis(5000)));

  std::atomic<bool> stop_dashboard{false};
  unsigned garbage_seed = 1;
  std::thread dashboard([&] {
    while (!stop_dashboard.load()) {
      const std::string page = http_get(lighthouse->port(), "/status");
      if (!page.empty() && page.find("200") == std::string::npos) fail("dashboard did not answer 200");
      garbage_client(lighthouse->port(), garbage_seed++);
      std::this_thread::sleep_for(Millis(3));
    }
  });

  const int leaving_group = groups - 1;
  const int leave_after = rounds / 2;
  std::vector<std::thread> workers;
  for (int g = 0; g < groups; ++g) {
    for (int r = 0; r < ranks; ++r) {
      workers.emplace_back([&, g, r] {
        try {
          ManagerClient client(managers[g]->address(), Millis(5000));
          int64_t step = 0;
          const int my_rounds = (g == leaving_group && groups > 1) ? leave_after : rounds;
          for (int round = 0; round < my_rounds; ++round) {
            const auto q = client.quorum(r, step, "meta" + std::to_string(r), false, Millis(20000));
            if (q.replica_world_size < 1 || q.replica_world_size > groups) fail("impossible replica_world_size");
            if (q.replica_rank < 0 || q.replica_rank >= q.replica_world_size) fail("replica_rank out of range");
            if (q.max_step < step) fail("max_step went backwards");
            if (client.checkpoint_metadata(r, Millis(5000)) != "meta" + std::to_string(r)) fail("metadata mix-up");
            // one rank of one group votes no every fifth round: the whole group must see false
            const bool group_vote_no = (round % 5 == 4);
            const bool my_vote = !(group_vote_no && r == 0);
            const bool decision = client.should_commit(r, step, my_vote, Millis(20000));
            if (decision != !group_vote_no) fail("should_commit decision differs from the AND of the votes");
            if (decision) ++step;
          }
        } catch (const std::exception& e) {
          fail(std::string("worker exception: ") + e.what());
        }
      });
    }
  }
  // the leaving group's workers finish first; take its server down while the others keep going
  if (groups > 1) {
    for (int r = 0; r < ranks; ++r) workers[leaving_group * ranks + r].join();
    managers[leaving_group]->shutdown();
    managers[leaving_group].reset();
  }
  for (int g = 0; g < groups; ++g) {
    if (g == leaving_group && groups > 1) continue;
    for (int r = 0; r < ranks; ++r) workers[g * ranks + r].join();
  }
  stop_dashboard.store(true);
  dashboard.join();
  for (auto& m : managers)
    if (m) m->shutdown();
  managers.clear();
  lighthouse->shutdown();
  lighthouse.reset();
  const int failures = g_failures.load();
  std::fprintf(stderr, "stress: %d failure(s)\n", failures);
  return failures == 0 ? 0 : 1;
}
