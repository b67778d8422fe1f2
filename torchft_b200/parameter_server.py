"""Parameter-server building block on top of reconfigurable process groups.

A server owns a TCPStore and an HTTP endpoint.  ``GET /new_session`` hands out a fresh
store prefix; server (rank 0) and client (rank 1) then configure a two-rank process
group on it and talk through ordinary collectives.  Every session runs in its own
thread on the server; a failed session only loses that session.  The lighthouse is not
involved.  Subclasses provide ``new_process_group()`` and ``forward(session_id, pg)``.

Parity: the reference's ``torchft/parameter_server.py:31-195`` (prototype there, too).
Unlike the reference the session runs in a dedicated thread instead of occupying the
HTTP handler thread, and the server keeps a table of the sessions that are open.
"""

from __future__ import annotations

import json
import logging
import socket
import threading
import urllib.request
import uuid
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from http.server import BaseHTTPRequestHandler
from typing import Dict, Type

from torch.distributed import TCPStore

from torchft_b200.http import advertised_host, make_http_server
from torchft_b200.process_group import ProcessGroup

logger: logging.Logger = logging.getLogger(__name__)

_SESSION_PATH = "/new_session"
_SERVER_RANK, _CLIENT_RANK, _SESSION_WORLD = 0, 1, 2


@dataclass
class _Session:
    """One client's rendezvous point: an id and the store prefix both ends configure on."""

    store_addr: str
    ident: str = field(default_factory=lambda: str(uuid.uuid4()))

    def announcement(self) -> bytes:
        return (json.dumps({"session_id": self.ident, "store_addr": self.store_addr}) + "\n").encode()


def _handler_for(ps: "ParameterServer") -> Type[BaseHTTPRequestHandler]:
    """HTTP front end of one server: answers the session request, then hands the session to a thread."""

    class _Handler(BaseHTTPRequestHandler):
        def _reply(self, status: int, content_type: str, body: bytes) -> None:
            self.send_response(status)
            self.send_header("Content-type", content_type)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)
            self.wfile.flush()

        def do_GET(self) -> None:  # noqa: N802 - http.server API
            if self.path != _SESSION_PATH:
                self._reply(400, "text/plain", f"invalid path, got {self.path}".encode())
                return
            session = ps._open_session()
            self._reply(200, "application/json", session.announcement())
            ps._run_in_thread(session)

        def log_message(self, fmt: str, *args: object) -> None:
            logger.debug(fmt % args)

    return _Handler


class ParameterServer(ABC):
    def __init__(self, port: int, store_port: int = 0) -> None:
        """``port`` is the HTTP port and ``store_port`` the TCPStore port; 0 picks a free one for either."""
        self.store = TCPStore(host_name="0.0.0.0", port=store_port, is_master=True, wait_for_workers=False)
        self._host = advertised_host(socket.gethostname())
        self._sessions: Dict[str, _Session] = {}
        self._sessions_lock = threading.Lock()
        self._server = make_http_server(port, _handler_for(self))
        self._thread = threading.Thread(target=self._serve, daemon=True, name="tft_parameter_server")
        self._thread.start()
        logger.info(f"Started ParameterServer on {self.address()}...")

    # ------------------------------------------------------------------ to be provided by the subclass
    @classmethod
    @abstractmethod
    def new_process_group(cls) -> ProcessGroup:
        """Returns a new, not yet configured process group (server and client both call this)."""

    @abstractmethod
    def forward(self, session_id: str, pg: ProcessGroup) -> None:
        """Runs once per session in its own thread (server is rank 0, client rank 1).

        Loop inside for several operations per session.  On an exception the group is
        dropped and the client has to open a new session.
        """

    # ------------------------------------------------------------------ client side
    @classmethod
    def new_session(cls, address: str) -> ProcessGroup:
        """Opens a session at ``address`` and returns the configured group (the client is rank 1)."""
        with urllib.request.urlopen(address) as response:
            offer = json.load(response)
        logger.info(f"connecting to session {offer['session_id']} at {offer['store_addr']}")
        group = cls.new_process_group()
        group.configure(offer["store_addr"], rank=_CLIENT_RANK, world_size=_SESSION_WORLD)
        return group

    # ------------------------------------------------------------------ server side
    def address(self) -> str:
        """``http://host:port/new_session``"""
        return f"http://{self._host}:{self._server.socket.getsockname()[1]}{_SESSION_PATH}"

    def open_sessions(self) -> int:
        """Number of sessions whose ``forward`` has not returned yet."""
        with self._sessions_lock:
            return len(self._sessions)

    def shutdown(self) -> None:
        self._server.shutdown()
        self._server.server_close()

    def _serve(self) -> None:
        try:
            self._server.serve_forever()
        except Exception:  # noqa: BLE001
            logger.exception("got exception in parameter server")

    def _open_session(self) -> _Session:
        session = _Session(store_addr="")
        session.store_addr = f"{self._host}:{self.store.port}/session/{session.ident}"
        with self._sessions_lock:
            self._sessions[session.ident] = session
        logger.info(f"creating new session {session.ident}")
        return session

    def _run_in_thread(self, session: _Session) -> None:
        threading.Thread(
            target=self._handle_session,
            args=(session.ident, session.store_addr),
            daemon=True,
            name=f"tft_ps_session_{session.ident[:8]}",
        ).start()

    def _handle_session(self, session_id: str, store_addr: str) -> None:
        try:
            group = self.new_process_group()
            group.configure(store_addr, rank=_SERVER_RANK, world_size=_SESSION_WORLD)
            self.forward(session_id, group)
        except Exception:  # noqa: BLE001 - only this session is lost
            logger.exception(f"session {session_id} failed")
        finally:
            with self._sessions_lock:
                self._sessions.pop(session_id, None)
