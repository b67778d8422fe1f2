// Standalone lighthouse executable.
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "cli.h"

int main(int argc, char** argv) {
  std::vector<std::string> args(argv + 1, argv + argc);
  try {
    return tft::run_lighthouse(tft::parse_lighthouse_args(args));
  } catch (const std::invalid_argument& e) {
    std::fprintf(stderr, "%s\n", e.what());
    return 2;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "lighthouse failed: %s\n", e.what());
    return 1;
  }
}
