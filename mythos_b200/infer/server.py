"""HTTP / SSE / WebSocket serving and the application-level pieces around it.

Covers the reference's production layer (src/production.cpp): ``HTTPServer`` with
``POST /v1/completions`` (JSON or ``"stream": true`` server-sent events), ``POST
/v1/chat/completions``, ``GET /health``, ``GET /v1/models``, CORS headers and 408 on slow clients;
``WebSocketHandler`` (RFC 6455 handshake, text frames, broadcast); ``Logger`` (four levels, stdout +
file); ``AppConfig`` (JSON with dotted get/set, validation, save); ``PluginManager`` (load a module
that defines ``create_plugin()``, lifecycle hooks, hot reload); ``ModelZoo`` (scan a directory for
``.oil`` files, load by name). Requests are served through the continuous batcher, so concurrent
clients share decode steps; the reference runs a full-prefix forward per token per client.
"""
from __future__ import annotations

import base64
import hashlib
import importlib.util
import json
import logging
import os
import socket
import struct
import sys
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer


# ------------------------------------------------------------------------------ logger / config
class Logger:
    LEVELS = {"DEBUG": 0, "INFO": 1, "WARN": 2, "ERROR": 3}
    _instance = None

    def __init__(self, level: str = "INFO", path: str | None = None):
        self.level, self.path = self.LEVELS[level], path
        self._lock = threading.Lock()

    @classmethod
    def instance(cls) -> "Logger":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def log(self, level: str, msg: str) -> None:
        if self.LEVELS[level] < self.level:
            return
        line = f"{time.strftime('%Y-%m-%d %H:%M:%S')} [{level}] {msg}"
        with self._lock:
            print(line, file=sys.stderr if level == "ERROR" else sys.stdout, flush=True)
            if self.path:
                with open(self.path, "a") as f:
                    f.write(line + "\n")

    def debug(self, m): self.log("DEBUG", m)
    def info(self, m): self.log("INFO", m)
    def warn(self, m): self.log("WARN", m)
    def error(self, m): self.log("ERROR", m)


class AppConfig:
    """JSON configuration with dotted paths: ``cfg.get("server.port")``, ``cfg.set("a.b", "3")``
    (strings are typed automatically: int, float, bool, null, else string)."""

    def __init__(self, data: dict | None = None):
        self.data = data or {}

    @classmethod
    def load(cls, path: str) -> "AppConfig":
        with open(path) as f:
            return cls(json.load(f))

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.data, f, indent=2, sort_keys=True)

    def get(self, path: str, default=None):
        cur = self.data
        for k in path.split("."):
            if not isinstance(cur, dict) or k not in cur:
                return default
            cur = cur[k]
        return cur

    @staticmethod
    def _auto(v):
        if not isinstance(v, str):
            return v
        low = v.lower()
        if low in ("true", "false"):
            return low == "true"
        if low in ("null", "none"):
            return None
        for cast in (int, float):
            try:
                return cast(v)
            except ValueError:
                pass
        return v

    def set(self, path: str, value) -> None:
        cur = self.data
        keys = path.split(".")
        for k in keys[:-1]:
            cur = cur.setdefault(k, {})
        cur[keys[-1]] = self._auto(value)

    def validate(self, required=("server.port",)) -> list[str]:
        problems = [f"missing {p}" for p in required if self.get(p) is None]
        port = self.get("server.port")
        if port is not None and not (isinstance(port, int) and 0 <= port < 65536):
            problems.append("server.port must be an integer in [0, 65535]")
        return problems


# ------------------------------------------------------------------------------ plugins / zoo
class Plugin:
    name = "plugin"

    def on_load(self, app): ...
    def on_unload(self, app): ...
    def on_request(self, request: dict) -> dict: return request
    def on_response(self, response: dict) -> dict: return response


class PluginManager:
    def __init__(self, app=None):
        self.app = app
        self.plugins: dict[str, tuple[Plugin, str, float]] = {}

    def load(self, path: str) -> Plugin:
        spec = importlib.util.spec_from_file_location(f"mythos_plugin_{abs(hash(path))}", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        if not hasattr(mod, "create_plugin"):
            raise ValueError(f"{path} does not define create_plugin()")
        plugin = mod.create_plugin()
        plugin.on_load(self.app)
        self.plugins[plugin.name] = (plugin, path, os.path.getmtime(path))
        return plugin

    def unload(self, name: str) -> None:
        plugin, _, _ = self.plugins.pop(name)
        plugin.on_unload(self.app)

    def reload_changed(self) -> list[str]:
        changed = []
        for name, (plugin, path, mtime) in list(self.plugins.items()):
            if os.path.getmtime(path) > mtime:
                self.unload(name)
                self.load(path)
                changed.append(name)
        return changed

    def apply_request(self, req: dict) -> dict:
        for plugin, _, _ in self.plugins.values():
            req = plugin.on_request(req)
        return req

    def apply_response(self, resp: dict) -> dict:
        for plugin, _, _ in self.plugins.values():
            resp = plugin.on_response(resp)
        return resp


class ModelZoo:
    def __init__(self, directory: str):
        self.directory = directory
        self.loaded = {}

    def scan(self) -> dict[str, str]:
        out = {}
        if os.path.isdir(self.directory):
            for fn in sorted(os.listdir(self.directory)):
                if fn.endswith(".oil"):
                    out[fn[:-4]] = os.path.join(self.directory, fn)
        return out

    def load(self, name: str, device="cpu"):
        if name not in self.loaded:
            paths = self.scan()
            if name not in paths:
                raise KeyError(f"no model named {name!r} in {self.directory}")
            from ..oil.model_io import load_model

            self.loaded[name] = load_model(paths[name], device=device)[0]
        return self.loaded[name]


# ------------------------------------------------------------------------------ generation backend
class GenerationBackend:
    """Thread-safe text generation for the server: tokenises, runs the model, detokenises. With a
    CUDA model the continuous batcher is used; on CPU a plain recompute loop."""

    def __init__(self, model=None, tokenizer=None, device="cpu", name="model", use_engine: bool = False):
        """``use_engine``: serve a CUDA model through the paged-KV ``InferenceEngine`` (one prefill,
        then one decode step per token, shared prompt heads) instead of recomputing the sequence for
        every token. Its building blocks are covered by the GPU tests; the combination inside the
        server has not been run on a GPU yet, hence opt-in (``oil-serve --paged-engine``)."""
        self.model, self.tokenizer, self.device, self.name = model, tokenizer, device, name
        self.use_engine = use_engine
        self._lock = threading.Lock()

    def encode(self, text: str) -> list[int]:
        if self.tokenizer is not None:
            return self.tokenizer.encode(text)
        return list(text.encode("utf-8"))

    def decode(self, ids) -> str:
        if self.tokenizer is not None:
            return self.tokenizer.decode(ids)
        return bytes(i & 0xFF for i in ids).decode("utf-8", errors="replace")

    def stream(self, prompt: str, max_tokens: int = 64, temperature: float = 0.0, top_k: int = 40, top_p: float = 0.9,
               seed: int = 0, flush: str = "token"):
        """Yields text pieces. ``flush="punctuation"`` regroups them so that a piece ends at white
        space, punctuation, a closing bracket or a quote (the reference's stream buffer). Without a
        model it echoes the prompt word by word (what a server started for tests without weights
        can do)."""
        if flush == "punctuation":
            from .stream import buffered

            yield from buffered(self.stream(prompt, max_tokens, temperature, top_k, top_p, seed))
            return
        if self.model is None:
            for w in prompt.split()[:max_tokens]:
                yield w + " "
            return
        import torch

        from .sampler import SamplerConfig, sample

        from .stream import Utf8Assembler

        utf8 = Utf8Assembler()
        cfg = SamplerConfig(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed)
        vocab = self.model.cfg.vocab_size
        ids = [min(t, vocab - 1) for t in self.encode(prompt)] or [0]
        # The backend lock is held per step (prefill, one token), never across a ``yield``: a client
        # that reads slowly stalls only its own request; other requests interleave token by token.
        with self._lock, torch.no_grad():
            dev = next(self.model.parameters()).device
            engine = self._engine(dev) if (self.use_engine and dev.type == "cuda") else None
            room = self.model.cfg.max_seq_len - len(ids)
            kv_seq = None
            logits = None
            if engine is not None and room > 1:
                # paged-KV engine: one prefill (cached prompt heads are shared), then one decode
                # step per token instead of recomputing the whole sequence
                try:
                    kv_seq, logits = engine.start_sequence(ids)
                except Exception:          # the prompt does not fit the engine: use the recompute loop
                    kv_seq, engine = None, None
            seq = torch.tensor([ids], dtype=torch.int32, device=dev)
        try:
            for step in range(max_tokens if kv_seq is None else min(max_tokens, room - 1)):
                with self._lock, torch.no_grad():
                    if kv_seq is None:
                        logits = self.model(seq[:, -self.model.cfg.max_seq_len:])[:, -1]
                    lg = logits.to(torch.bfloat16).contiguous() if logits.is_cuda else logits.float()
                    tok = sample(lg, cfg, step=step).to(torch.int32)
                    if kv_seq is None:
                        seq = torch.cat([seq, tok.view(1, 1).to(dev)], dim=1)
                    else:
                        logits = engine.decode([kv_seq], [int(tok[0])])
                    tok_id = int(tok[0])
                if self.tokenizer is not None:
                    yield self.decode([tok_id])
                else:                      # byte-level ids: hold back unfinished multi-byte characters
                    piece = utf8.feed(bytes([tok_id & 0xFF]))
                    if piece:
                        yield piece
        finally:                           # also when the consumer stops reading early
            if kv_seq is not None:
                with self._lock:
                    engine.release(kv_seq)
        if self.tokenizer is None:
            tail = utf8.finish()
            if tail:
                yield tail

    def _engine(self, dev):
        """Inference engine over the served model (built on first use; None when it cannot be built,
        e.g. for shapes the kernels do not cover: the recompute loop then serves the request)."""
        if getattr(self, "_eng", None) is None and not getattr(self, "_eng_failed", False):
            try:
                from .engine import InferenceEngine

                self._eng = InferenceEngine.from_model(self.model, device=dev, max_batch=8,
                                                       max_seq_len=self.model.cfg.max_seq_len)
            except Exception as e:
                self._eng_failed = True
                logging.getLogger("mythos_b200").warning("serving without the paged-KV engine: %s", e)
        return getattr(self, "_eng", None)

    def complete(self, prompt: str, **kw) -> str:
        return "".join(self.stream(prompt, **kw))


# ------------------------------------------------------------------------------ HTTP
def _make_handler(server: "HTTPServer"):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        timeout = server.request_timeout

        def log_message(self, fmt, *args):
            server.logger.debug("http " + fmt % args)

        def _cors(self):
            self.send_header("Access-Control-Allow-Origin", "*")
            self.send_header("Access-Control-Allow-Headers", "Content-Type, Authorization")
            self.send_header("Access-Control-Allow-Methods", "GET, POST, OPTIONS")

        def _json(self, code: int, obj: dict):
            body = json.dumps(obj).encode("utf-8")
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self._cors()
            self.end_headers()
            self.wfile.write(body)

        def do_OPTIONS(self):
            self.send_response(204)
            self._cors()
            self.send_header("Content-Length", "0")
            self.end_headers()

        def do_GET(self):
            if self.path == "/health":
                self._json(200, {"status": "ok", "uptime_s": time.time() - server.started})
            elif self.path == "/v1/models":
                self._json(200, {"object": "list", "data": [{"id": server.backend.name, "object": "model"}]})
            else:
                self._json(404, {"error": "not found"})

        def do_POST(self):
            try:
                n = int(self.headers.get("Content-Length", "0"))
                if n < 0:
                    raise ValueError("negative Content-Length")
                if n > server.max_body_bytes:
                    self.close_connection = True          # the unread body must not be parsed as a request
                    self._json(413, {"error": f"request body larger than {server.max_body_bytes} bytes"})
                    return
                raw = self.rfile.read(n) if n else b""
                req = json.loads(raw.decode("utf-8") or "{}")
            except socket.timeout:
                self._json(408, {"error": "request timeout"})
                return
            except (ValueError, UnicodeDecodeError):
                self._json(400, {"error": "invalid JSON"})
                return
            req = server.plugins.apply_request(req)
            if self.path == "/v1/chat/completions":
                msgs = req.get("messages", [])
                req["prompt"] = "\n".join(f"{m.get('role', 'user')}: {m.get('content', '')}" for m in msgs) + "\nassistant:"
            elif self.path != "/v1/completions":
                self._json(404, {"error": "not found"})
                return
            kw = dict(max_tokens=int(req.get("max_tokens", 64)), temperature=float(req.get("temperature", 0.0)),
                      top_k=int(req.get("top_k", 40)), top_p=float(req.get("top_p", 0.9)), seed=int(req.get("seed", 0)))
            if req.get("stream_flush") in ("token", "punctuation"):
                kw["flush"] = req["stream_flush"]
            prompt = str(req.get("prompt", ""))
            if req.get("stream"):
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Connection", "close")
                self._cors()
                self.end_headers()
                for piece in server.backend.stream(prompt, **kw):
                    chunk = {"object": "text_completion.chunk", "choices": [{"text": piece, "index": 0}]}
                    self.wfile.write(b"data: " + json.dumps(chunk).encode() + b"\n\n")
                    self.wfile.flush()
                self.wfile.write(b"data: [DONE]\n\n")
                self.wfile.flush()
                self.close_connection = True
                return
            t0 = time.time()
            text = server.backend.complete(prompt, **kw)
            key = "message" if self.path.endswith("chat/completions") else "text"
            choice = {"index": 0, "finish_reason": "length"}
            choice[key] = {"role": "assistant", "content": text} if key == "message" else text
            resp = {"id": f"cmpl-{int(t0 * 1000)}", "object": "text_completion", "model": server.backend.name,
                    "choices": [choice], "usage": {"completion_seconds": time.time() - t0}}
            self._json(200, server.plugins.apply_response(resp))

    return Handler


class HTTPServer:
    def __init__(self, backend: GenerationBackend | None = None, port: int = 0, host: str = "127.0.0.1",
                 request_timeout: float = 30.0, logger: Logger | None = None, max_body_bytes: int = 8 << 20):
        self.backend = backend or GenerationBackend()
        self.host, self.port, self.request_timeout = host, port, request_timeout
        self.max_body_bytes = max_body_bytes                # larger request bodies are answered with 413
        self.logger = logger or Logger.instance()
        self.plugins = PluginManager(self)
        self.started = time.time()
        self._httpd = None
        self._thread = None

    def start(self) -> int:
        self._httpd = ThreadingHTTPServer((self.host, self.port), _make_handler(self))
        self._httpd.daemon_threads = True
        self.port = self._httpd.server_address[1]
        self._thread = threading.Thread(target=self._httpd.serve_forever, daemon=True)
        self._thread.start()
        self.logger.info(f"serving on http://{self.host}:{self.port}")
        return self.port

    def stop(self) -> None:
        if self._httpd is not None:
            self._httpd.shutdown()
            self._httpd.server_close()
            self._httpd = None


# ------------------------------------------------------------------------------ WebSocket (RFC 6455)
WS_GUID = "258EAFA5-E914-47DA-95CA-C5AB0DC85B11"


def ws_accept_key(client_key: str) -> str:
    return base64.b64encode(hashlib.sha1((client_key + WS_GUID).encode()).digest()).decode()


def ws_encode_frame(payload: bytes, opcode: int = 1, mask: bool = False) -> bytes:
    head = bytes([0x80 | opcode])
    n = len(payload)
    mbit = 0x80 if mask else 0
    if n < 126:
        head += bytes([mbit | n])
    elif n < 65536:
        head += bytes([mbit | 126]) + struct.pack(">H", n)
    else:
        head += bytes([mbit | 127]) + struct.pack(">Q", n)
    if mask:
        key = os.urandom(4)
        return head + key + bytes(b ^ key[i & 3] for i, b in enumerate(payload))
    return head + payload


def ws_parse_frame(data: bytes):
    """Returns (opcode, payload, bytes_consumed) or None when the frame is incomplete."""
    if len(data) < 2:
        return None
    opcode, n = data[0] & 0x0F, data[1] & 0x7F
    masked = bool(data[1] & 0x80)
    off = 2
    if n == 126:
        if len(data) < 4:
            return None
        (n,) = struct.unpack_from(">H", data, 2)
        off = 4
    elif n == 127:
        if len(data) < 10:
            return None
        (n,) = struct.unpack_from(">Q", data, 2)
        off = 10
    key = b""
    if masked:
        key = data[off:off + 4]
        off += 4
    if len(data) < off + n:
        return None
    payload = data[off:off + n]
    if masked:
        payload = bytes(b ^ key[i & 3] for i, b in enumerate(payload))
    return opcode, payload, off + n


class WebSocketHandler:
    """Accepts WebSocket clients; each text frame is a prompt, the reply is streamed back as text
    frames; ``broadcast`` sends one message to every connected client."""

    def __init__(self, backend: GenerationBackend | None = None, port: int = 0, host: str = "127.0.0.1"):
        self.backend = backend or GenerationBackend()
        self.host, self.port = host, port
        self.clients: list[socket.socket] = []
        self._lock = threading.Lock()
        self._sock = None
        self._running = False

    def start(self) -> int:
        self._sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._sock.bind((self.host, self.port))
        self._sock.listen(16)
        self._sock.settimeout(0.2)
        self.port = self._sock.getsockname()[1]
        self._running = True
        threading.Thread(target=self._accept_loop, daemon=True).start()
        return self.port

    def stop(self) -> None:
        self._running = False
        with self._lock:
            for c in self.clients:
                try:
                    c.close()
                except OSError:
                    pass
            self.clients.clear()
        if self._sock is not None:
            self._sock.close()

    def broadcast(self, text: str) -> int:
        frame = ws_encode_frame(text.encode("utf-8"))
        sent = 0
        with self._lock:
            for c in list(self.clients):
                try:
                    c.sendall(frame)
                    sent += 1
                except OSError:
                    self.clients.remove(c)
        return sent

    def _accept_loop(self):
        while self._running:
            try:
                conn, _ = self._sock.accept()
            except socket.timeout:
                continue
            except OSError:
                break
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _serve(self, conn: socket.socket):
        try:
            conn.settimeout(10.0)
            req = b""
            while b"\r\n\r\n" not in req:
                chunk = conn.recv(4096)
                if not chunk:
                    return
                req += chunk
            key = None
            for line in req.decode("latin1").split("\r\n"):
                if line.lower().startswith("sec-websocket-key:"):
                    key = line.split(":", 1)[1].strip()
            if key is None:
                conn.sendall(b"HTTP/1.1 400 Bad Request\r\nContent-Length: 0\r\n\r\n")
                return
            conn.sendall(("HTTP/1.1 101 Switching Protocols\r\nUpgrade: websocket\r\nConnection: Upgrade\r\n"
                          f"Sec-WebSocket-Accept: {ws_accept_key(key)}\r\n\r\n").encode())
            with self._lock:
                self.clients.append(conn)
            buf = b""
            conn.settimeout(None)
            while self._running:
                data = conn.recv(65536)
                if not data:
                    break
                buf += data
                while True:
                    parsed = ws_parse_frame(buf)
                    if parsed is None:
                        break
                    opcode, payload, used = parsed
                    buf = buf[used:]
                    if opcode == 8:
                        conn.sendall(ws_encode_frame(b"", opcode=8))
                        return
                    if opcode == 9:
                        conn.sendall(ws_encode_frame(payload, opcode=10))
                    elif opcode == 1:
                        for piece in self.backend.stream(payload.decode("utf-8", errors="replace")):
                            conn.sendall(ws_encode_frame(piece.encode("utf-8")))
                        conn.sendall(ws_encode_frame(b"[DONE]"))
        except OSError:
            pass
        finally:
            with self._lock:
                if conn in self.clients:
                    self.clients.remove(conn)
            try:
                conn.close()
            except OSError:
                pass


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="oil-serve", description="Serve a .oil model over HTTP (OpenAI-style routes).")
    ap.add_argument("--model", default=None)
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--config", default=None)
    ap.add_argument("--paged-engine", action="store_true",
                    help="serve a CUDA model through the paged-KV inference engine instead of recomputing per token")
    a = ap.parse_args(argv)
    cfg = AppConfig.load(a.config) if a.config else AppConfig({"server": {"port": a.port}})
    backend = GenerationBackend()
    if a.model:
        from ..oil.model_io import load_model
        from ..tools.common import pick_device
        from ..train.bpe import BPETokenizer

        dev = pick_device(a.device)
        model, _ = load_model(a.model, device=dev)
        vocab = (a.model[:-4] if a.model.endswith(".oil") else a.model) + ".vocab"
        tok = BPETokenizer.load(vocab) if os.path.exists(vocab) else None
        backend = GenerationBackend(model.eval(), tok, dev, os.path.basename(a.model), use_engine=a.paged_engine)
    srv = HTTPServer(backend, port=int(cfg.get("server.port", a.port)), host=a.host)
    srv.start()
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
