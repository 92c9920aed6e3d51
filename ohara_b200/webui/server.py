"""Standard-library HTTP server that streams chat replies as Server-Sent Events.

Protocol (same as the reference server, ohara/webui/server.py:29-218):

* ``GET /`` and ``GET /static/*``: the single-page UI (paths are resolved inside the static
  directory; anything that escapes it is a 404).
* ``GET /api/info`` → ``{"model": <ChatEngine.metadata>, "defaults": <SamplingConfig>}``.
* ``POST /api/chat`` with ``{messages, temperature?, top_p?, top_k?, max_new_tokens?, seed?}`` →
  ``text/event-stream`` over chunked transfer: ``data: {"delta": ...}`` frames, then
  ``data: {"done": true}`` (or ``data: {"error": "Type: message"}``), then the zero-length chunk.
  Validation failures are a JSON 400.

One model and one KV cache are shared, so generation is serialised behind a lock.
"""

from __future__ import annotations

import json
import mimetypes
import threading
from dataclasses import asdict
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path
from typing import Any

from ohara_b200.chat_engine import ChatEngine, SamplingConfig

STATIC_DIR = Path(__file__).parent / "static"
MAX_REQUEST_BYTES = 4 * 1024 * 1024
_ROLES = {"user", "assistant", "system"}


class BadRequest(ValueError):
    """Client error that should be reported as HTTP 400."""


def parse_chat_request(payload: Any, defaults: SamplingConfig):
    """Validate a ``/api/chat`` body; returns ``(messages, SamplingConfig, seed)``."""
    if not isinstance(payload, dict):
        raise BadRequest("request body must be a JSON object")
    messages = payload.get("messages")
    if not isinstance(messages, list) or not messages:
        raise BadRequest("'messages' must be a non-empty list")
    for message in messages:
        if not isinstance(message, dict):
            raise BadRequest("each message must be an object")
        if message.get("role") not in _ROLES:
            raise BadRequest(f"unsupported role: {message.get('role')!r}")
        if not isinstance(message.get("content"), str):
            raise BadRequest("message content must be a string")
    try:
        sampling = SamplingConfig(
            temperature=float(payload.get("temperature", defaults.temperature)),
            top_p=float(payload.get("top_p", defaults.top_p)),
            top_k=int(payload.get("top_k", defaults.top_k)),
            max_new_tokens=int(payload.get("max_new_tokens", defaults.max_new_tokens)),
        )
        seed = payload.get("seed")
        seed = int(seed) if seed is not None else None
    except (TypeError, ValueError) as error:
        raise BadRequest(str(error)) from error
    return messages, sampling, seed


class ChatRequestHandler(BaseHTTPRequestHandler):
    server_version = "ohara-b200-webui"
    protocol_version = "HTTP/1.1"

    # bound by create_server
    engine: ChatEngine
    generation_lock: threading.Lock
    checkpoint_path: str | None
    default_sampling: SamplingConfig

    def log_message(self, format: str, *args: Any) -> None:  # keep the console for training logs
        return

    # -- plumbing ----------------------------------------------------------------------------
    def _send(self, body: bytes, content_type: str, status: int = 200) -> None:
        self.send_response(status)
        self.send_header("Content-Type", content_type)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def _send_json(self, payload: dict[str, Any], status: int = 200) -> None:
        self._send(json.dumps(payload).encode("utf-8"), "application/json", status)

    def _not_found(self) -> None:
        self._send_json({"error": "not found"}, status=404)

    def _read_json(self) -> Any:
        length = int(self.headers.get("Content-Length") or 0)
        if length <= 0:
            raise BadRequest("request body is empty")
        if length > MAX_REQUEST_BYTES:
            raise BadRequest("request body is too large")
        try:
            return json.loads(self.rfile.read(length).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            # (the parser's own message, as the reference replies)
            raise BadRequest(str(error)) from error

    def _serve_static(self, relative: str) -> None:
        root = STATIC_DIR.resolve()
        target = (STATIC_DIR / relative).resolve()
        if root != target and root not in target.parents:
            return self._not_found()
        if not target.is_file():
            return self._not_found()
        kind, _ = mimetypes.guess_type(target.name)
        self._send(target.read_bytes(), kind or "application/octet-stream")

    def _chunk(self, data: bytes) -> None:
        self.wfile.write(f"{len(data):X}\r\n".encode("ascii") + data + b"\r\n")
        self.wfile.flush()

    def _event(self, payload: dict[str, Any]) -> None:
        self._chunk(f"data: {json.dumps(payload)}\n\n".encode("utf-8"))

    # -- routes ------------------------------------------------------------------------------
    def do_GET(self) -> None:  # noqa: N802
        path = self.path.split("?", 1)[0]
        if path in ("/", "/index.html"):
            self._serve_static("index.html")
        elif path.startswith("/static/"):
            self._serve_static(path[len("/static/"):])
        elif path == "/api/info":
            self._send_json({"model": self.engine.metadata(self.checkpoint_path),
                             "defaults": asdict(self.default_sampling)})
        else:
            self._not_found()

    def do_POST(self) -> None:  # noqa: N802
        if self.path.split("?", 1)[0] != "/api/chat":
            return self._not_found()
        try:
            messages, sampling, seed = parse_chat_request(self._read_json(), self.default_sampling)
        except BadRequest as error:
            return self._send_json({"error": str(error)}, status=400)
        self.send_response(200)
        self.send_header("Content-Type", "text/event-stream")
        self.send_header("Cache-Control", "no-cache")
        self.send_header("X-Accel-Buffering", "no")
        self.send_header("Transfer-Encoding", "chunked")
        self.end_headers()
        gone = (BrokenPipeError, ConnectionResetError)
        try:
            with self.generation_lock:
                for delta in self.engine.generate_stream(messages, sampling, seed=seed):
                    self._event({"delta": delta})
            self._event({"done": True})
        except gone:
            return
        except Exception as error:  # noqa: BLE001 - shown in the UI instead of a dead stream
            try:
                self._event({"error": f"{type(error).__name__}: {error}"})
            except gone:
                return
        finally:
            try:
                self._chunk(b"")
            except gone:
                pass


def create_server(engine: ChatEngine, *, host: str = "127.0.0.1", port: int = 8080,
                  checkpoint_path: str | None = None,
                  sampling: SamplingConfig | None = None) -> ThreadingHTTPServer:
    """Build (without starting) a server bound to ``host:port`` (port 0 picks a free one)."""
    handler = type("BoundChatRequestHandler", (ChatRequestHandler,), {
        "engine": engine,
        "generation_lock": threading.Lock(),
        "checkpoint_path": checkpoint_path,
        "default_sampling": sampling or SamplingConfig(),
    })
    return ThreadingHTTPServer((host, port), handler)


def serve(engine: ChatEngine, *, host: str = "127.0.0.1", port: int = 8080,
          checkpoint_path: str | None = None, sampling: SamplingConfig | None = None) -> None:
    server = create_server(engine, host=host, port=port, checkpoint_path=checkpoint_path,
                           sampling=sampling)
    shown = "localhost" if host in ("0.0.0.0", "127.0.0.1") else host
    print(f"ohara_b200 chat UI on http://{shown}:{server.server_address[1]}  (ctrl-c to stop)")
    try:
        server.serve_forever()
    except KeyboardInterrupt:
        print("\nshutting down")
    finally:
        server.shutdown()
        server.server_close()
