// Python bindings of the control plane (module torchft_b200._control).
// Classes and signatures follow the reference's torchft/torchft.pyi: Manager,
// ManagerClient, Lighthouse, QuorumResult, lighthouse_main.  Every blocking call
// releases the GIL.  RPC failures map to TimeoutError (cancelled / deadline exceeded)
// or RuntimeError (everything else).
#include <pybind11/chrono.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <csignal>

#include "cli.h"
#include "h2.h"
#include "lighthouse.h"
#include "manager.h"
#include "quorum.h"

namespace py = pybind11;
using namespace tft;

namespace {

struct QuorumResult {
  int64_t quorum_id = 0;
  int64_t replica_rank = 0;
  int64_t replica_world_size = 1;
  std::string recover_src_manager_address;
  std::optional<int64_t> recover_src_rank;
  std::vector<int64_t> recover_dst_ranks;
  std::string store_address;
  int64_t max_step = 0;
  std::optional<int64_t> max_rank;
  int64_t max_world_size = 1;
  bool heal = false;
};

QuorumResult to_result(const wire::ManagerQuorumResponse& r) {
  QuorumResult q;
  q.quorum_id = r.quorum_id;
  q.replica_rank = r.replica_rank;
  q.replica_world_size = r.replica_world_size;
  q.recover_src_manager_address = r.recover_src_manager_address;
  q.recover_src_rank = r.recover_src_rank;
  q.recover_dst_ranks = r.recover_dst_ranks;
  q.store_address = r.store_address;
  q.max_step = r.max_step;
  q.max_rank = r.max_rank;
  q.max_world_size = r.max_world_size;
  q.heal = r.heal;
  return q;
}

net::Millis to_ms(std::chrono::duration<double> d) {
  return net::Millis(static_cast<long long>(d.count() * 1000.0 + 0.5));
}

[[noreturn]] void rethrow(const net::RpcError& e) {
  if (e.is_timeout()) {
    PyErr_SetString(PyExc_TimeoutError, e.what());
  } else {
    PyErr_SetString(PyExc_RuntimeError, e.what());
  }
  throw py::error_already_set();
}

template <typename F>
auto guarded(F&& f) -> decltype(f()) {
  try {
    py::gil_scoped_release release;
    return f();
  } catch (const net::RpcError& e) {
    rethrow(e);
  }
}

wire::QuorumMember member_from_dict(const py::dict& d) {
  wire::QuorumMember m;
  if (d.contains("replica_id")) m.replica_id = d["replica_id"].cast<std::string>();
  if (d.contains("address")) m.address = d["address"].cast<std::string>();
  if (d.contains("store_address")) m.store_address = d["store_address"].cast<std::string>();
  if (d.contains("step")) m.step = d["step"].cast<int64_t>();
  if (d.contains("world_size")) m.world_size = d["world_size"].cast<uint64_t>();
  if (d.contains("shrink_only")) m.shrink_only = d["shrink_only"].cast<bool>();
  if (d.contains("force_reconfigure")) m.force_reconfigure = d["force_reconfigure"].cast<bool>();
  return m;
}

py::dict member_to_dict(const wire::QuorumMember& m) {
  py::dict d;
  d["replica_id"] = m.replica_id;
  d["address"] = m.address;
  d["store_address"] = m.store_address;
  d["step"] = m.step;
  d["world_size"] = m.world_size;
  d["shrink_only"] = m.shrink_only;
  return d;
}

py::dict quorum_to_dict(const wire::Quorum& q) {
  py::dict d;
  d["quorum_id"] = q.quorum_id;
  py::list members;
  for (const auto& m : q.participants) members.append(member_to_dict(m));
  d["participants"] = members;
  d["created"] = static_cast<double>(q.created.seconds) + q.created.nanos * 1e-9;
  return d;
}

}  // namespace

#ifndef TFT_MODULE_NAME
#define TFT_MODULE_NAME _control
#endif
// TFT_MODULE_NAME lets the same bindings be built under another module name.
PYBIND11_MODULE(TFT_MODULE_NAME, m) {
  m.doc() = "C++ control plane: lighthouse, manager server and clients";

  py::class_<QuorumResult>(m, "QuorumResult", py::module_local())
      .def(py::init<>())
      .def_readwrite("quorum_id", &QuorumResult::quorum_id)
      .def_readwrite("replica_rank", &QuorumResult::replica_rank)
      .def_readwrite("replica_world_size", &QuorumResult::replica_world_size)
      .def_readwrite("recover_src_manager_address", &QuorumResult::recover_src_manager_address)
      .def_readwrite("recover_src_rank", &QuorumResult::recover_src_rank)
      .def_readwrite("recover_dst_ranks", &QuorumResult::recover_dst_ranks)
      .def_readwrite("store_address", &QuorumResult::store_address)
      .def_readwrite("max_step", &QuorumResult::max_step)
      .def_readwrite("max_rank", &QuorumResult::max_rank)
      .def_readwrite("max_world_size", &QuorumResult::max_world_size)
      .def_readwrite("heal", &QuorumResult::heal);

  py::class_<ManagerServer>(m, "Manager", py::module_local())
      .def(py::init([](const std::string& replica_id, const std::string& lighthouse_addr, const std::string& hostname,
                       const std::string& bind, const std::string& store_addr, uint64_t world_size,
                       std::chrono::duration<double> heartbeat_interval, std::chrono::duration<double> connect_timeout) {
             try {
               py::gil_scoped_release release;
               return std::make_unique<ManagerServer>(replica_id, lighthouse_addr, hostname, bind, store_addr,
                                                      world_size, to_ms(heartbeat_interval), to_ms(connect_timeout));
             } catch (const net::RpcError& e) {
               rethrow(e);
             }
           }),
           py::arg("replica_id"), py::arg("lighthouse_addr"), py::arg("hostname"), py::arg("bind"),
           py::arg("store_addr"), py::arg("world_size"), py::arg("heartbeat_interval"), py::arg("connect_timeout"))
      .def("address", &ManagerServer::address)
      .def("shutdown", [](ManagerServer& s) {
        py::gil_scoped_release release;
        s.shutdown();
      });

  py::class_<ManagerClient>(m, "ManagerClient", py::module_local())
      .def(py::init([](const std::string& addr, std::chrono::duration<double> connect_timeout) {
             try {
               py::gil_scoped_release release;
               return std::make_unique<ManagerClient>(addr, to_ms(connect_timeout));
             } catch (const net::RpcError& e) {
               rethrow(e);
             }
           }),
           py::arg("addr"), py::arg("connect_timeout"))
      .def("quorum",
           [](ManagerClient& c, int64_t rank, int64_t step, const std::string& checkpoint_metadata, bool shrink_only,
              std::chrono::duration<double> timeout, bool force_reconfigure) {
             return guarded([&] {
               return to_result(c.quorum(rank, step, checkpoint_metadata, shrink_only, to_ms(timeout), force_reconfigure));
             });
           },
           py::arg("rank"), py::arg("step"), py::arg("checkpoint_metadata"), py::arg("shrink_only"),
           py::arg("timeout"), py::arg("force_reconfigure") = false)
      .def("checkpoint_metadata",
           [](ManagerClient& c, int64_t rank, std::chrono::duration<double> timeout) {
             return guarded([&] { return c.checkpoint_metadata(rank, to_ms(timeout)); });
           },
           py::arg("rank"), py::arg("timeout"))
      .def("should_commit",
           [](ManagerClient& c, int64_t rank, int64_t step, bool should_commit, std::chrono::duration<double> timeout) {
             return guarded([&] { return c.should_commit(rank, step, should_commit, to_ms(timeout)); });
           },
           py::arg("rank"), py::arg("step"), py::arg("should_commit"), py::arg("timeout"))
      .def("kill",
           [](ManagerClient& c, const std::string& msg, std::chrono::duration<double> timeout) {
             guarded([&] { c.kill(msg, to_ms(timeout)); return 0; });
           },
           py::arg("msg"), py::arg("timeout"));

  py::class_<LighthouseClient>(m, "LighthouseClient", py::module_local())
      .def(py::init([](const std::string& addr, std::chrono::duration<double> connect_timeout) {
             try {
               py::gil_scoped_release release;
               return std::make_unique<LighthouseClient>(addr, to_ms(connect_timeout));
             } catch (const net::RpcError& e) {
               rethrow(e);
             }
           }),
           py::arg("addr"), py::arg("connect_timeout"))
      .def("quorum",
           [](LighthouseClient& c, const py::dict& requester, std::chrono::duration<double> timeout) {
             wire::QuorumMember me = member_from_dict(requester);
             wire::Quorum q = guarded([&] { return c.quorum(me, to_ms(timeout)); });
             return quorum_to_dict(q);
           },
           py::arg("requester"), py::arg("timeout"))
      .def("heartbeat",
           [](LighthouseClient& c, const std::string& replica_id, std::chrono::duration<double> timeout) {
             guarded([&] { c.heartbeat(replica_id, to_ms(timeout)); return 0; });
           },
           py::arg("replica_id"), py::arg("timeout") = std::chrono::duration<double>(5.0));

  py::class_<Lighthouse>(m, "Lighthouse", py::module_local())
      .def(py::init([](const std::string& bind, uint64_t min_replicas, std::optional<uint64_t> join_timeout_ms,
                       std::optional<uint64_t> quorum_tick_ms, std::optional<uint64_t> heartbeat_timeout_ms) {
             LighthouseOptions opt;
             opt.bind = bind;
             opt.min_replicas = min_replicas;
             opt.join_timeout_ms = join_timeout_ms.value_or(100);
             opt.quorum_tick_ms = quorum_tick_ms.value_or(100);
             opt.heartbeat_timeout_ms = heartbeat_timeout_ms.value_or(5000);
             py::gil_scoped_release release;
             return std::make_unique<Lighthouse>(opt);
           }),
           py::arg("bind"), py::arg("min_replicas"), py::arg("join_timeout_ms") = py::none(),
           py::arg("quorum_tick_ms") = py::none(), py::arg("heartbeat_timeout_ms") = py::none())
      .def("address", &Lighthouse::address)
      .def("shutdown", [](Lighthouse& l) {
        py::gil_scoped_release release;
        l.shutdown();
      });

  m.def("lighthouse_main", [](std::optional<std::vector<std::string>> argv) {
    std::vector<std::string> args;
    if (argv) {
      args = *argv;
    } else {
      py::list sys_argv = py::module_::import("sys").attr("argv");
      for (size_t i = 1; i < sys_argv.size(); ++i) args.push_back(sys_argv[i].cast<std::string>());
    }
    LighthouseOptions opt;
    try {
      opt = parse_lighthouse_args(args);
    } catch (const std::invalid_argument& e) {
      throw py::value_error(e.what());
    }
    std::signal(SIGINT, SIG_DFL);  // let ctrl-C end the blocking native loop
    py::gil_scoped_release release;
    run_lighthouse(opt);
  }, py::arg("argv") = py::none());

  // ---- pure functions, exposed so their rules can be tested table-driven from Python
  m.def("quorum_compute",
        [](double now_s, const py::dict& state, uint64_t min_replicas, uint64_t join_timeout_ms,
           uint64_t heartbeat_timeout_ms) {
          // Times are seconds on an arbitrary monotonic axis.
          auto tp = [](double s) {
            return net::Clock::time_point(std::chrono::duration_cast<net::Clock::duration>(
                std::chrono::duration<double>(s + 1.0e6)));
          };
          LighthouseState st;
          if (state.contains("participants")) {
            for (auto item : state["participants"].cast<py::dict>()) {
              py::dict d = item.second.cast<py::dict>();
              MemberDetails md;
              md.joined = tp(d["joined"].cast<double>());
              md.member = member_from_dict(d["member"].cast<py::dict>());
              st.participants[item.first.cast<std::string>()] = md;
            }
          }
          if (state.contains("heartbeats"))
            for (auto item : state["heartbeats"].cast<py::dict>())
              st.heartbeats[item.first.cast<std::string>()] = tp(item.second.cast<double>());
          if (state.contains("prev_quorum") && !state["prev_quorum"].is_none()) {
            py::dict pq = state["prev_quorum"].cast<py::dict>();
            wire::Quorum q;
            q.quorum_id = pq.contains("quorum_id") ? pq["quorum_id"].cast<int64_t>() : 0;
            for (auto mem : pq["participants"].cast<py::list>()) q.participants.push_back(member_from_dict(mem.cast<py::dict>()));
            st.prev_quorum = q;
          }
          LighthouseOptions opt;
          opt.min_replicas = min_replicas;
          opt.join_timeout_ms = join_timeout_ms;
          opt.heartbeat_timeout_ms = heartbeat_timeout_ms;
          auto res = quorum_compute(tp(now_s), st, opt);
          py::object members = py::none();
          if (res.first) {
            py::list l;
            for (const auto& mem : *res.first) l.append(member_to_dict(mem));
            members = l;
          }
          return py::make_tuple(members, res.second);
        },
        py::arg("now"), py::arg("state"), py::arg("min_replicas"), py::arg("join_timeout_ms") = 60000,
        py::arg("heartbeat_timeout_ms") = 5000);

  m.def("quorum_changed", [](const py::list& a, const py::list& b) {
    std::vector<wire::QuorumMember> va, vb;
    for (auto x : a) va.push_back(member_from_dict(x.cast<py::dict>()));
    for (auto x : b) vb.push_back(member_from_dict(x.cast<py::dict>()));
    return quorum_changed(va, vb);
  });

  m.def("compute_quorum_results",
        [](const std::string& replica_id, int64_t rank, int64_t quorum_id, const py::list& participants) {
          wire::Quorum q;
          q.quorum_id = quorum_id;
          for (auto x : participants) q.participants.push_back(member_from_dict(x.cast<py::dict>()));
          try {
            return to_result(compute_quorum_results(replica_id, rank, q));
          } catch (const net::RpcError& e) {
            rethrow(e);
          }
        },
        py::arg("replica_id"), py::arg("rank"), py::arg("quorum_id"), py::arg("participants"));

  m.def("parse_grpc_timeout", [](const std::string& s) -> py::object {
    auto d = net::parse_grpc_timeout(s);
    if (!d) return py::none();
    return py::float_(std::chrono::duration<double>(*d).count());
  });

  m.def("retry_backoff_probe",
        [](int fail_times, uint64_t initial_ms, std::optional<uint64_t> timeout_ms, std::optional<int> max_retries) {
          net::BackoffOptions opt;
          opt.initial = net::Millis(initial_ms);
          opt.max_jitter = net::Millis(0);
          if (timeout_ms) opt.timeout = net::Millis(*timeout_ms);
          opt.max_retries = max_retries;
          int attempts = 0;
          bool ok;
          {
            py::gil_scoped_release release;
            ok = net::retry_backoff(opt, [&](int attempt) { return attempt >= fail_times; }, &attempts);
          }
          return py::make_tuple(ok, attempts);
        },
        py::arg("fail_times"), py::arg("initial_ms") = 1, py::arg("timeout_ms") = py::none(),
        py::arg("max_retries") = py::none());

  m.def("set_log_enabled", &net::set_log_enabled);

  // Wire protocol of the clients created afterwards: "framed" (default) or "grpc" (HTTP/2, the
  // reference's format).  Servers accept both on the same port at all times.
  m.def("set_rpc_protocol", [](const std::string& name) {
    try {
      net::set_rpc_protocol(name);
    } catch (const std::invalid_argument& e) {
      throw py::value_error(e.what());
    }
  });
  m.def("rpc_protocol", &net::rpc_protocol);

  // HPACK pieces, exposed for tests against RFC 7541 vectors and other HTTP/2 stacks.
  m.def("huffman_encode", [](const py::bytes& b) { return py::bytes(net::h2::huffman_encode(std::string(b))); });
  m.def("huffman_decode", [](const py::bytes& b) -> py::object {
    const std::string in(b);
    std::string out;
    if (!net::h2::huffman_decode(reinterpret_cast<const uint8_t*>(in.data()), in.size(), &out)) return py::none();
    return py::bytes(out);
  });
  m.def("hpack_encode", [](const std::vector<std::pair<std::string, std::string>>& headers, bool huffman) {
    std::vector<net::h2::Header> hs;
    for (const auto& kv : headers) hs.push_back({kv.first, kv.second});
    return py::bytes(net::h2::hpack_encode(hs, huffman));
  }, py::arg("headers"), py::arg("huffman") = true);
  py::class_<net::h2::HpackDecoder>(m, "HpackDecoder", py::module_local())
      .def(py::init<>())
      .def("decode", [](net::h2::HpackDecoder& self, const py::bytes& block) -> py::object {
        std::vector<net::h2::Header> out;
        if (!self.decode(std::string(block), &out)) return py::none();
        py::list result;
        for (const auto& h : out) result.append(py::make_tuple(py::bytes(h.name), py::bytes(h.value)));
        return result;
      });

  // Wire codec round trips for interop tests against other protobuf implementations.
  m.def("encode_manager_quorum_response", [](const QuorumResult& r) {
    wire::ManagerQuorumResponse w;
    w.quorum_id = r.quorum_id; w.recover_src_manager_address = r.recover_src_manager_address;
    w.recover_src_rank = r.recover_src_rank; w.recover_dst_ranks = r.recover_dst_ranks;
    w.store_address = r.store_address; w.max_step = r.max_step; w.max_rank = r.max_rank;
    w.max_world_size = r.max_world_size; w.replica_rank = r.replica_rank;
    w.replica_world_size = r.replica_world_size; w.heal = r.heal;
    return py::bytes(w.encode());
  });
  m.def("decode_manager_quorum_response", [](const py::bytes& b) {
    return to_result(wire::ManagerQuorumResponse::decode(std::string(b)));
  });
  m.def("encode_quorum_member", [](const py::dict& d) { return py::bytes(member_from_dict(d).encode()); });
  m.def("decode_quorum_member", [](const py::bytes& b) { return member_to_dict(wire::QuorumMember::decode(std::string(b))); });
}
