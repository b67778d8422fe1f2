"""Threaded HTTP server that listens on the IPv6 wildcard (dual stack where available)."""

import socket
from http.server import ThreadingHTTPServer


class _IPv6HTTPServer(ThreadingHTTPServer):
    address_family = socket.AF_INET6
    request_queue_size = 1024
    daemon_threads = True


class _IPv4HTTPServer(ThreadingHTTPServer):
    request_queue_size = 1024
    daemon_threads = True


def make_http_server(port: int, handler: type) -> ThreadingHTTPServer:
    """Binds ``[::]:port`` and falls back to ``0.0.0.0`` on hosts without IPv6."""
    try:
        return _IPv6HTTPServer(("::", port), handler)
    except OSError:
        return _IPv4HTTPServer(("0.0.0.0", port), handler)


def advertised_host(hostname: str) -> str:
    """``hostname`` if it resolves from here, else the loopback address."""
    try:
        socket.getaddrinfo(hostname, None)
        return hostname
    except OSError:
        return "127.0.0.1"
