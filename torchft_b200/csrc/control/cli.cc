#include "cli.h"

#include <chrono>
#include <stdexcept>
#include <thread>

#include "lighthouse.h"

namespace tft {

LighthouseOptions parse_lighthouse_args(const std::vector<std::string>& args) {
  LighthouseOptions opt;
  bool have_min = false;
  const std::string usage =
      "usage: tft_lighthouse --min_replicas N [--bind [::]:29510] [--join_timeout_ms 60000] "
      "[--quorum_tick_ms 100] [--heartbeat_timeout_ms 5000]";
  for (size_t i = 0; i < args.size(); ++i) {
    std::string key = args[i];
    std::string value;
    auto eq = key.find('=');
    if (eq != std::string::npos) {
      value = key.substr(eq + 1);
      key = key.substr(0, eq);
    } else if (key == "--help" || key == "-h") {
      throw std::invalid_argument(usage);
    } else {
      if (i + 1 >= args.size()) throw std::invalid_argument("missing value for " + key + "\n" + usage);
      value = args[++i];
    }
    for (auto& c : key) if (c == '-' && &c - &key[0] >= 2) c = '_';
    try {
      if (key == "--bind") opt.bind = value;
      else if (key == "--join_timeout_ms") opt.join_timeout_ms = std::stoull(value);
      else if (key == "--min_replicas") { opt.min_replicas = std::stoull(value); have_min = true; }
      else if (key == "--quorum_tick_ms") opt.quorum_tick_ms = std::stoull(value);
      else if (key == "--heartbeat_timeout_ms") opt.heartbeat_timeout_ms = std::stoull(value);
      else throw std::invalid_argument("unknown flag " + key + "\n" + usage);
    } catch (const std::invalid_argument&) {
      throw;
    } catch (const std::exception&) {
      throw std::invalid_argument("invalid value for " + key + ": " + value);
    }
  }
  if (!have_min) throw std::invalid_argument("--min_replicas is required\n" + usage);
  return opt;
}

int run_lighthouse(const LighthouseOptions& opt) {
  Lighthouse lighthouse(opt);
  while (true) std::this_thread::sleep_for(std::chrono::seconds(3600));
  return 0;
}

}  // namespace tft
