"""Serving layer on CPU: HTTP routes (JSON, SSE, CORS, errors), WebSocket handshake and frames,
config, plugins, model zoo, scheduler / batching policies, speculative decoding, beam search,
tokenizer, metrics writers, importers, planner, eval metrics."""
import http.client
import json
import socket
import struct
import time

import numpy as np
import pytest
import torch

from mythos_b200.models import DenseModel, TransformerConfig


def _tiny():
    torch.manual_seed(0)
    return DenseModel(TransformerConfig(vocab_size=256, hidden_size=32, num_layers=1, num_heads=2, head_dim=16,
                                        ffn_hidden_size=64, max_seq_len=64, oil_block_size=32, weight_format="fp32"))


def test_http_server_routes_and_streaming():
    from mythos_b200.infer.server import GenerationBackend, HTTPServer

    srv = HTTPServer(GenerationBackend(_tiny(), None, "cpu", "tiny"), port=0)
    port = srv.start()
    try:
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
        c.request("GET", "/health")
        r = c.getresponse()
        assert r.status == 200 and json.loads(r.read())["status"] == "ok"
        assert r.getheader("Access-Control-Allow-Origin") == "*"
        c.request("GET", "/v1/models")
        assert json.loads(c.getresponse().read())["data"][0]["id"] == "tiny"
        c.request("POST", "/v1/completions", json.dumps({"prompt": "ab", "max_tokens": 3}),
                  {"Content-Type": "application/json"})
        body = json.loads(c.getresponse().read())
        assert isinstance(body["choices"][0]["text"], str)
        c.request("POST", "/v1/chat/completions", json.dumps({"messages": [{"role": "user", "content": "hi"}],
                                                               "max_tokens": 2}))
        assert "message" in json.loads(c.getresponse().read())["choices"][0]
        c.request("POST", "/v1/completions", "{not json")
        r = c.getresponse()
        r.read()
        assert r.status == 400
        c.request("GET", "/nope")
        r = c.getresponse()
        r.read()
        assert r.status == 404
        c2 = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
        c2.request("POST", "/v1/completions", json.dumps({"prompt": "ab", "max_tokens": 3, "stream": True}))
        r = c2.getresponse()
        assert r.getheader("Content-Type") == "text/event-stream"
        events = [l for l in r.read().decode().split("\n\n") if l.startswith("data: ")]
        assert events[-1] == "data: [DONE]" and len(events) == 4
    finally:
        srv.stop()


def test_http_server_starts_without_a_model_on_port_zero():
    from mythos_b200.infer.server import HTTPServer

    srv = HTTPServer(None, port=0)
    port = srv.start()
    assert port > 0
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    c.request("POST", "/v1/completions", json.dumps({"prompt": "echo these words", "max_tokens": 2}))
    assert json.loads(c.getresponse().read())["choices"][0]["text"] == "echo these "
    srv.stop()


def test_http_server_rejects_oversized_and_negative_bodies_and_interleaves_streams():
    import socket

    from mythos_b200.infer.server import GenerationBackend, HTTPServer

    backend = GenerationBackend(_tiny(), None, "cpu", "tiny")
    srv = HTTPServer(backend, port=0, max_body_bytes=1024)
    port = srv.start()
    try:
        for length, want in ((5000, b"413"), (-5, b"400")):
            s = socket.create_connection(("127.0.0.1", port), timeout=10)
            s.sendall(f"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Length: {length}\r\n\r\n".encode())
            assert want in s.recv(4096).split(b"\r\n")[0]        # answered without waiting for a body
            s.close()
        # a generator that has yielded its first piece does not hold the backend lock
        slow = backend.stream("ab", max_tokens=4)
        next(slow)
        assert backend._lock.acquire(timeout=1.0)
        backend._lock.release()
        assert isinstance(backend.complete("cd", max_tokens=2), str)   # a second request runs to the end meanwhile
        assert len(list(slow)) >= 1
    finally:
        srv.stop()


def test_websocket_handshake_frames_and_broadcast():
    from mythos_b200.infer import server as S

    assert S.ws_accept_key("dGhlIHNhbXBsZSBub25jZQ==") == "s3pPLMBiTxaQ9kYGzzhZRbK+xOo="  # RFC 6455 example
    for n in (5, 200, 70000):
        payload = bytes(i % 251 for i in range(n))
        op, out, used = S.ws_parse_frame(S.ws_encode_frame(payload, opcode=2, mask=True))
        assert op == 2 and out == payload and used > n
    assert S.ws_parse_frame(b"\x81") is None
    ws = S.WebSocketHandler(None, port=0)
    port = ws.start()
    try:
        s = socket.create_connection(("127.0.0.1", port), timeout=10)
        s.sendall(b"GET / HTTP/1.1\r\nHost: x\r\nUpgrade: websocket\r\nConnection: Upgrade\r\n"
                  b"Sec-WebSocket-Key: dGhlIHNhbXBsZSBub25jZQ==\r\nSec-WebSocket-Version: 13\r\n\r\n")
        resp = s.recv(4096).decode()
        assert "101 Switching Protocols" in resp and "s3pPLMBiTxaQ9kYGzzhZRbK+xOo=" in resp
        time.sleep(0.1)
        assert ws.broadcast("hello") == 1
        op, payload, _ = S.ws_parse_frame(s.recv(4096))
        assert op == 1 and payload == b"hello"
        s.sendall(S.ws_encode_frame(b"two words", mask=True))
        got = b""
        while b"[DONE]" not in got:
            got += s.recv(4096)
        s.close()
    finally:
        ws.stop()


def test_app_config_plugins_zoo_logger(tmp_path):
    from mythos_b200.infer.server import AppConfig, Logger, ModelZoo, PluginManager
    from mythos_b200.oil.model_io import save_model

    cfg = AppConfig()
    cfg.set("server.port", "8080")
    cfg.set("model.temperature", "0.7")
    cfg.set("flags.stream", "true")
    assert cfg.get("server.port") == 8080 and cfg.get("model.temperature") == 0.7 and cfg.get("flags.stream") is True
    assert cfg.get("missing.key", 5) == 5 and cfg.validate() == []
    cfg.set("server.port", "99999")
    assert cfg.validate()
    p = str(tmp_path / "cfg.json")
    cfg.save(p)
    assert AppConfig.load(p).get("flags.stream") is True
    plug = tmp_path / "plug.py"
    plug.write_text("from mythos_b200.infer.server import Plugin\n"
                    "class P(Plugin):\n    name='upper'\n"
                    "    def on_request(self, r):\n        r['prompt']=r.get('prompt','').upper(); return r\n"
                    "def create_plugin():\n    return P()\n")
    pm = PluginManager()
    pm.load(str(plug))
    assert pm.apply_request({"prompt": "abc"})["prompt"] == "ABC"
    pm.unload("upper")
    assert pm.apply_request({"prompt": "abc"})["prompt"] == "abc"
    save_model(_tiny(), str(tmp_path / "tiny.oil"))
    zoo = ModelZoo(str(tmp_path))
    assert list(zoo.scan()) == ["tiny"]
    assert zoo.load("tiny").cfg.hidden_size == 32
    with pytest.raises(KeyError):
        zoo.load("absent")
    log = Logger("WARN", str(tmp_path / "log.txt"))
    log.info("hidden")
    log.error("shown")
    assert "shown" in (tmp_path / "log.txt").read_text() and "hidden" not in (tmp_path / "log.txt").read_text()


def test_scheduler_batcher_and_decoding_strategies():
    from mythos_b200.infer.serving import (DynamicBatcher, Request, RequestScheduler, SpeculativeDecoder, beam_search,
                                           compute_logprobs)

    sch = RequestScheduler()
    sch.push(Request([1], priority=0))
    sch.push(Request([2], priority=5))
    sch.push(Request([3], priority=5, deadline=time.time() + 100))
    sch.push(Request([4], priority=9, deadline=time.time() - 1))  # already expired
    assert [sch.pop().prompt for _ in range(3)] == [[3], [2], [1]]
    for i in range(5):
        sch.push(Request([0] * 10, max_new_tokens=10))
    assert len(DynamicBatcher(max_batch=8, max_tokens=45).take(sch)) == 2
    m = _tiny()
    spec = SpeculativeDecoder(m, m, gamma=3)
    out = spec.generate([1, 2, 3], 6, temperature=0.0)
    seq, want = [1, 2, 3], []
    for _ in range(6):
        t = int(m(torch.tensor([seq], dtype=torch.int32))[0, -1].argmax())
        want.append(t)
        seq.append(t)
    assert out == want and spec.stats["accepted"] == spec.stats["proposed"]
    beams = beam_search(m, [1, 2], 3, beams=3)
    assert len(beams) == 3 and beams[0][1] >= beams[1][1] and len(beams[0][0]) == 3
    lp = compute_logprobs(m, [1, 2, 3, 4, 5])
    assert lp.shape == (4,) and bool((lp <= 0).all())


def test_tokenizer_metrics_importers_planner_eval(tmp_path):
    from mythos_b200.eval import compute_bleu, compute_rouge_l, eval_classification, eval_perplexity
    from mythos_b200.oil import importers, planner
    from mythos_b200.train.bpe import BPETokenizer
    from mythos_b200.train.metrics import EventWriter, JsonlLogger, masked_crc32c, read_events

    text = "low lower lowest newer newest wide wider widest " * 50
    tok = BPETokenizer()
    tok.train(text, 300)
    ids = tok.encode("lower newest")
    assert tok.decode(ids) == "lower newest" and len(ids) < len("lower newest") and tok.vocab_size <= 300
    p = str(tmp_path / "t.vocab")
    tok.save(p)
    raw = open(p, "rb").read()
    assert struct.unpack_from("<i", raw, 0)[0] == tok.vocab_size and raw[4:9] == struct.pack("<i", 1) + b"\x00"
    assert BPETokenizer.load(p).encode("lower newest") == ids
    w = EventWriter(str(tmp_path / "tb"))
    w.write_event("loss", 1.25, 7)
    w.close()
    payloads = list(read_events(w.path))
    assert len(payloads) == 2 and b"loss" in payloads[1] and struct.pack("<f", 1.25) in payloads[1]
    assert masked_crc32c(b"") == ((0 >> 15 | 0 << 17) + 0xA282EAD8) & 0xFFFFFFFF
    jl = JsonlLogger("proj", "run", str(tmp_path))
    jl.log({"loss": 2.0}, step=1)
    jl.close()
    assert json.loads(open(jl.path).read())["loss"] == 2.0
    importers.write_safetensors(str(tmp_path / "a.safetensors"), {"w": np.arange(6, dtype=np.float32).reshape(2, 3)})
    assert importers.read_safetensors(str(tmp_path / "a.safetensors"))["w"].shape == (2, 3)
    # a minimal GGUF v3 file with one F32 and one Q8_0 tensor
    def s(x): return struct.pack("<Q", len(x)) + x
    vals = np.arange(32, dtype=np.float32) / 10
    d = np.float16(np.abs(vals).max() / 127)
    q = np.clip(np.rint(vals / np.float32(d)), -127, 127).astype(np.int8)
    infos = s(b"a") + struct.pack("<I", 1) + struct.pack("<Q", 4) + struct.pack("<I", 0) + struct.pack("<Q", 0)
    infos += s(b"b") + struct.pack("<I", 1) + struct.pack("<Q", 32) + struct.pack("<I", 8) + struct.pack("<Q", 32)
    head = struct.pack("<IIQQ", 0x46554747, 3, 2, 0) + infos
    head += b"\0" * ((-len(head)) % 32)
    data = np.arange(4, dtype="<f4").tobytes() + b"\0" * 16 + d.tobytes() + q.tobytes()
    (tmp_path / "m.gguf").write_bytes(head + data)
    tensors, _ = importers.read_gguf(str(tmp_path / "m.gguf"))
    assert np.array_equal(tensors["a"], np.arange(4, dtype=np.float32))
    assert np.allclose(tensors["b"], vals, atol=float(d))
    wt = torch.randn(32, 256) * 0.02
    fmts, bpw = planner.plan(wt, 1.5, 256)
    assert abs(bpw - 1.5) <= 0.1 and len(fmts) == 32
    mix = planner.compute_format_mix(1000, 1.58 * 0.95 + 8 * 0.01 + 4 * 0.04)
    assert sum(mix.values()) == 1000
    deq, blocks = planner.quantize_mixed(wt, fmts, 256)
    assert deq.shape == wt.shape and len(blocks) == 32
    assert compute_bleu([1, 2, 3, 4, 5], [1, 2, 3, 4, 5]) == pytest.approx(1.0)
    assert compute_bleu([9, 9, 9, 9], [1, 2, 3, 4]) == 0.0
    assert compute_rouge_l([1, 2, 3, 9], [1, 2, 3, 4]) == pytest.approx(0.75)
    assert eval_classification([0, 1, 1], [0, 1, 0])["accuracy"] == pytest.approx(2 / 3)
    r = eval_perplexity(_tiny(), torch.randint(0, 256, (90,)), context=32, stride=16)
    assert r["tokens"] == 89 and r["perplexity"] > 1


def test_stream_buffer_flushes_at_breaks_and_keeps_the_tail():
    from mythos_b200.infer.stream import StreamBuffer, Utf8Assembler, buffered

    got = []
    buf = StreamBuffer(got.append)
    for piece in ["Hel", "lo", ",", " wor", "ld", "!", " (ok", ")", " tail"]:
        buf.append(piece)
    assert got == ["Hello,", " world!", " (ok)"]
    buf.close()
    assert got[-1] == " tail" and buf.buffer == ""
    assert list(buffered(iter(["a", "b ", "c"]))) == ["ab ", "c"]
    long = StreamBuffer(got.append, max_chars=4)
    long.append("abcdef")
    assert got[-1] == "abcdef"
    # a multi-byte character split over two chunks comes out whole
    asm = Utf8Assembler()
    raw = "naïve ☃".encode("utf-8")
    text = "".join(asm.feed(raw[i:i + 1]) for i in range(len(raw))) + asm.finish()
    assert text == "naïve ☃"
    assert Utf8Assembler().feed(b"\xe2\x98") == ""


def test_backend_stream_regroups_at_punctuation():
    from mythos_b200.infer.server import GenerationBackend

    be = GenerationBackend()                      # no model: echoes the prompt word by word
    plain = list(be.stream("one two, three", max_tokens=8))
    grouped = list(be.stream("one two, three", max_tokens=8, flush="punctuation"))
    assert "".join(plain) == "".join(grouped)
    assert all(g[-1] in " ,.!?" for g in grouped)


def test_reduced_precision_activation_wrappers_pool_and_stream_config():
    import torch.nn as nn

    from mythos_b200.infer.extras import (DecodeResult, FP8Inference, INT8Inference, InferenceMemoryPool, StreamConfig,
                                          decode_with_config, fake_quant_fp8, fake_quant_int8, quantize_per_token_int8)

    torch.manual_seed(0)
    x = torch.randn(6, 64) * 3
    q, s = quantize_per_token_int8(x)
    assert q.dtype == torch.int8 and s.shape == (6, 1) and int(q.abs().max()) == 127
    assert float((fake_quant_int8(x) - x).abs().max()) <= float(s.max()) * 0.5 + 1e-6
    assert float((fake_quant_fp8(x) - x).abs().max()) <= 0.07 * float(x.abs().max())      # e4m3: 3 mantissa bits
    assert torch.equal(fake_quant_int8(torch.zeros(2, 8)), torch.zeros(2, 8))
    net = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), nn.Linear(32, 8))
    ref = net(x).detach()
    for cls, tol in ((INT8Inference, 0.05), (FP8Inference, 0.15)):
        w = cls(net)
        y = w(x)
        assert w.is_quantized and w.layers_seen == 2
        err = float((y - ref).abs().max())
        assert 0 < err < tol * float(ref.abs().max())
    assert not any(m._forward_pre_hooks for m in net.modules())          # hooks are gone after the call

    pool = InferenceMemoryPool(256, 3)
    a, b, c = pool.alloc(), pool.alloc(), pool.alloc()
    assert pool.used == 3 and pool.capacity == 3 and a.numel() == 256
    with pytest.raises(MemoryError):
        pool.alloc()
    pool.free(b)
    assert pool.used == 2 and pool.alloc().data_ptr() == b.data_ptr()
    with pytest.raises(ValueError):
        pool.free(torch.empty(256, dtype=torch.uint8))

    text = "ab\ncdSTOPef"
    vocab = sorted(set(text)) + ["<eos>"]

    def step(ids):                                  # a model that recites `text`, then emits <eos>
        k = len(ids) - 1
        lg = torch.full((len(vocab),), -5.0)
        lg[vocab.index(text[k]) if k < len(text) else len(vocab) - 1] = 5.0
        return lg

    detok = lambda ids: "".join(vocab[i] for i in ids)
    pieces = []
    r = decode_with_config(step, [0], StreamConfig(stream=True, max_tokens=50, eos_id=len(vocab) - 1), detok, pieces.append)
    assert isinstance(r, DecodeResult) and r.text == text and r.finish_reason == "eos" and "".join(pieces) == text
    assert len(r.logprobs) == len(text) and 1.0 <= r.perplexity < 1.01
    assert decode_with_config(step, [0], StreamConfig(max_tokens=50, stop_on_newline=True), detok).text == "ab\n"
    r = decode_with_config(step, [0], StreamConfig(max_tokens=50, stop_sequences=["STOP"]), detok)
    assert r.text == "ab\ncd" and r.finish_reason == "stop"
    assert decode_with_config(step, [0], StreamConfig(max_tokens=4), detok).finish_reason == "length"
