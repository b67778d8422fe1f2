"""Parameter-server building block on top of reconfigurable process groups.

A server owns a TCPStore and an HTTP endpoint.  ``GET /new_session`` hands out a fresh
store prefix; server (rank 0) and client (rank 1) then configure a two-rank process
group on it and talk through ordinary collectives.  Every session runs in its own
thread on the server; a failed session only loses that session.  The lighthouse is not
involved.  Subclasses provide ``new_process_group()`` and ``forward(session_id, pg)``.

Parity: the reference's ``torchft/parameter_server.py:31-195`` (prototype there, too).
Unlike the reference the session runs in a dedicated thread instead of occupying the
HTTP handler thread.
"""

from __future__ import annotations

import json
import logging
import socket
import threading
import urllib.request
import uuid
from abc import ABC, abstractmethod
from http.server import BaseHTTPRequestHandler

from torch.distributed import TCPStore

from torchft_b200.http import advertised_host, make_http_server
from torchft_b200.process_group import ProcessGroup

logger: logging.Logger = logging.getLogger(__name__)


class ParameterServer(ABC):
    def __init__(self, port: int, store_port: int = 0) -> None:
        """
        Args:
            port: HTTP port (0 picks a free one)
            store_port: TCPStore port (0 picks a free one)
        """
        self.store = TCPStore(host_name="0.0.0.0", port=store_port, is_master=True, wait_for_workers=False)
        ps = self

        class RequestHandler(BaseHTTPRequestHandler):
            def do_GET(self) -> None:  # noqa: N802 - http.server API
                if self.path != "/new_session":
                    self.send_response(400)
                    self.send_header("Content-type", "text/plain")
                    self.end_headers()
                    self.wfile.write(f"invalid path, got {self.path}".encode())
                    return
                session_id = str(uuid.uuid4())
                host = advertised_host(socket.gethostname())
                store_addr = f"{host}:{ps.store.port}/session/{session_id}"
                logger.info(f"creating new session {session_id}")
                body = (json.dumps({"session_id": session_id, "store_addr": store_addr}) + "\n").encode()
                self.send_response(200)
                self.send_header("Content-type", "application/json")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
                self.wfile.flush()
                threading.Thread(
                    target=ps._handle_session,
                    args=(session_id, store_addr),
                    daemon=True,
                    name=f"tft_ps_session_{session_id[:8]}",
                ).start()

            def log_message(self, fmt: str, *args: object) -> None:
                logger.debug(fmt % args)

        self._server = make_http_server(port, RequestHandler)
        logger.info(f"Started ParameterServer on {self.address()}...")
        self._thread = threading.Thread(target=self._serve, daemon=True, name="tft_parameter_server")
        self._thread.start()

    def address(self) -> str:
        """``http://host:port/new_session``"""
        port = self._server.socket.getsockname()[1]
        return f"http://{advertised_host(socket.gethostname())}:{port}/new_session"

    def shutdown(self) -> None:
        self._server.shutdown()
        self._server.server_close()

    def _serve(self) -> None:
        try:
            self._server.serve_forever()
        except Exception:  # noqa: BLE001
            logger.exception("got exception in parameter server")

    @classmethod
    @abstractmethod
    def new_process_group(cls) -> ProcessGroup:
        """Returns a new, not yet configured process group (server and client both call this)."""

    @classmethod
    def new_session(cls, address: str) -> ProcessGroup:
        """Client side: opens a session at ``address`` and returns the configured group (client is rank 1)."""
        with urllib.request.urlopen(address) as f:
            data = json.load(f)
        session_id = data["session_id"]
        store_addr = data["store_addr"]
        logger.info(f"connecting to session {session_id} at {store_addr}")
        pg = cls.new_process_group()
        pg.configure(store_addr, rank=1, world_size=2)
        return pg

    def _handle_session(self, session_id: str, store_addr: str) -> None:
        try:
            pg = self.new_process_group()
            pg.configure(store_addr, rank=0, world_size=2)
            self.forward(session_id, pg)
        except Exception:  # noqa: BLE001 - only this session is lost
            logger.exception(f"session {session_id} failed")

    @abstractmethod
    def forward(self, session_id: str, pg: ProcessGroup) -> None:
        """Runs once per session in its own thread (server is rank 0, client rank 1).

        Loop inside for several operations per session.  On an exception the group is
        dropped and the client has to open a new session.
        """
