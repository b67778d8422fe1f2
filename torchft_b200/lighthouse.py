"""``python -m torchft_b200.lighthouse --min_replicas N [--bind [::]:29510] [--join_timeout_ms 60000]
[--quorum_tick_ms 100] [--heartbeat_timeout_ms 5000]``

Runs the C++ lighthouse in this process until interrupted (same flags as the reference's
``torchft_lighthouse`` console script; the stand-alone binary
``torchft_b200/lib/tft_lighthouse`` takes the same flags).
"""

import sys

from torchft_b200._control import lighthouse_main


def main() -> None:
    try:
        lighthouse_main(sys.argv[1:])
    except ValueError as e:
        print(e, file=sys.stderr)
        sys.exit(2)


if __name__ == "__main__":
    main()
