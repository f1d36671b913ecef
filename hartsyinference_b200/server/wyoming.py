"""Wyoming protocol endpoint for wake-word detection (the protocol voice satellites speak).

A message is one JSON line ``{"type": ..., "data": {...}, "data_length": n, "payload_length": m}``
followed by ``n`` bytes of further JSON data (merged over ``data``) and ``m`` bytes of payload.
The wake service understands:

* ``describe``  -> ``info`` listing the loaded wake words;
* ``detect`` ``{"names": [...]}``  restricts the session to those words (all when absent);
* ``audio-start`` / ``audio-chunk`` (PCM payload; ``rate``, ``width``, ``channels`` in the data) /
  ``audio-stop``; chunks are mixed to mono, resampled to 16 kHz and pushed through the session's
  :class:`~hartsyinference_b200.audio.wake.WakeDetector`;
* it answers ``detection`` ``{"name", "timestamp"}`` (milliseconds into the stream) when a word
  fires, and ``not-detected`` after ``audio-stop`` if none did.

Every connection is its own stream with its own detector state; the models are shared.
Reference: src/HartsyInference.Engine/Audio/Wake/Wyoming/ (WyomingFrameCodec, WyomingConnection,
WyomingListener, WyomingInfo), WakeSession.cs, WakeListener.cs; the CLI's wake-client.
"""
from __future__ import annotations

import asyncio
import json
from typing import Optional

import torch

from ..audio.wake import RATE, WakeModelSet
from ..audio.wav import resample

VERSION = "1.5.2"
MAX_HEADER, MAX_DATA, MAX_PAYLOAD = 64 * 1024, 1 << 20, 8 << 20


def encode_event(kind: str, data: Optional[dict] = None, payload: bytes = b"") -> bytes:
    header = {"type": kind, "version": VERSION}
    extra = b""
    if data:
        extra = json.dumps(data, separators=(",", ":")).encode()
        header["data_length"] = len(extra)
    if payload:
        header["payload_length"] = len(payload)
    return json.dumps(header, separators=(",", ":")).encode() + b"\n" + extra + payload


async def read_event(reader: asyncio.StreamReader):
    """-> (type, data, payload), or None at end of stream. Oversized or malformed frames raise ValueError."""
    line = await reader.readline()
    if not line:
        return None
    if len(line) > MAX_HEADER:
        raise ValueError("header line too long")
    try:
        header = json.loads(line)
    except json.JSONDecodeError as e:
        raise ValueError(f"malformed header: {e}") from None
    if not isinstance(header, dict) or not isinstance(header.get("type"), str):
        raise ValueError("header without a type")
    data = dict(header.get("data") or {})
    n, m = int(header.get("data_length") or 0), int(header.get("payload_length") or 0)
    if not (0 <= n <= MAX_DATA and 0 <= m <= MAX_PAYLOAD):
        raise ValueError("frame exceeds the size limits")
    if n:
        more = json.loads(await reader.readexactly(n))
        if isinstance(more, dict):
            data.update(more)
    payload = await reader.readexactly(m) if m else b""
    return header["type"], data, payload


def pcm_to_mono16k(payload: bytes, rate: int, width: int, channels: int) -> torch.Tensor:
    """PCM bytes -> mono float samples in int16 scale at 16 kHz."""
    if width == 2:
        x = torch.frombuffer(bytearray(payload[:len(payload) // 2 * 2]), dtype=torch.int16).float()
    elif width == 4:
        x = torch.frombuffer(bytearray(payload[:len(payload) // 4 * 4]), dtype=torch.int32).float() / 65536.0
    elif width == 1:
        x = (torch.frombuffer(bytearray(payload), dtype=torch.uint8).float() - 128.0) * 256.0
    else:
        raise ValueError(f"unsupported sample width {width}")
    if channels > 1:
        x = x[:x.numel() // channels * channels].view(-1, channels).mean(1)
    if rate != RATE and x.numel():
        x = resample(x, rate, RATE)
    return x


class WakeSession:
    """One connection's stream: detector state, the selected words, the stream clock."""

    def __init__(self, models: WakeModelSet, settings: Optional[dict] = None):
        self.models, self.detector = models, models.detector(settings)
        self.fired = False

    def select(self, names) -> None:
        if names:
            for w in self.detector.words:
                if w not in names:
                    self.detector.remove_word(w)

    def start(self) -> None:
        self.detector.reset()
        self.fired = False

    def push(self, payload: bytes, rate: int, width: int, channels: int) -> list[dict]:
        out = []
        for d in self.detector.push(pcm_to_mono16k(payload, rate, width, channels)):
            self.fired = True
            out.append({"name": d.word, "timestamp": int(d.sample_index * 1000 / RATE), "score": round(d.score, 4)})
        return out


def info_event(models: WakeModelSet) -> bytes:
    attribution = {"name": "hartsyinference_b200", "url": ""}
    words = [{"name": n, "description": n.replace("_", " "), "attribution": attribution, "installed": True, "languages": ["en"],
              "phrase": n.replace("_", " "), "version": None} for n in models.heads]
    return encode_event("info", {"wake": [{"name": "hartsyinference_b200", "description": "wake-word detection", "attribution": attribution,
                                          "installed": True, "version": VERSION, "models": words}],
                                 "asr": [], "tts": [], "handle": [], "intent": [], "satellite": None})


class WyomingWakeServer:
    def __init__(self, models: WakeModelSet, host: str = "127.0.0.1", port: int = 10400, settings: Optional[dict] = None):
        self.models, self.host, self.port, self.settings = models, host, port, settings
        self._server: Optional[asyncio.AbstractServer] = None
        self.sessions = 0

    async def _handle(self, reader: asyncio.StreamReader, writer: asyncio.StreamWriter) -> None:
        session = WakeSession(self.models, self.settings)
        self.sessions += 1
        loop = asyncio.get_running_loop()
        try:
            while True:
                event = await read_event(reader)
                if event is None:
                    break
                kind, data, payload = event
                if kind == "describe":
                    writer.write(info_event(self.models))
                elif kind == "detect":
                    session.select(data.get("names"))
                elif kind == "audio-start":
                    session.start()
                elif kind == "audio-chunk":
                    args = (payload, int(data.get("rate", RATE)), int(data.get("width", 2)), int(data.get("channels", 1)))
                    for hit in await loop.run_in_executor(None, session.push, *args):      # the models run off the event loop
                        writer.write(encode_event("detection", hit))
                elif kind == "audio-stop":
                    if not session.fired:
                        writer.write(encode_event("not-detected"))
                elif kind == "ping":
                    writer.write(encode_event("pong", data))
                await writer.drain()
        except (ValueError, asyncio.IncompleteReadError, ConnectionError):
            pass                                      # a broken frame ends this connection only
        finally:
            self.sessions -= 1
            writer.close()

    async def start(self) -> int:
        self._server = await asyncio.start_server(self._handle, self.host, self.port)
        self.port = self._server.sockets[0].getsockname()[1]
        return self.port

    async def stop(self) -> None:
        if self._server is not None:
            self._server.close()
            await self._server.wait_closed()

    def serve_forever(self) -> None:
        async def main():
            await self.start()
            async with self._server:
                await self._server.serve_forever()
        asyncio.run(main())


async def stream_wav(host: str, port: int, samples: torch.Tensor, rate: int, names=None, chunk_ms: int = 80,
                     realtime: bool = False) -> list[dict]:
    """The satellite's side: sends ``samples`` (float, +-1) as 16-bit PCM chunks and collects the answers."""
    reader, writer = await asyncio.open_connection(host, port)
    fmt = {"rate": rate, "width": 2, "channels": 1}
    hits: list[dict] = []
    try:
        if names:
            writer.write(encode_event("detect", {"names": list(names)}))
        writer.write(encode_event("audio-start", {**fmt, "timestamp": 0}))
        pcm = (samples.float().clamp(-1, 1) * 32767.0).round().to(torch.int16)
        step = max(1, rate * chunk_ms // 1000)
        for i in range(0, pcm.numel(), step):
            writer.write(encode_event("audio-chunk", {**fmt, "timestamp": int(i * 1000 / rate)}, pcm[i:i + step].numpy().tobytes()))
            await writer.drain()
            if realtime:
                await asyncio.sleep(chunk_ms / 1000)
        writer.write(encode_event("audio-stop", {"timestamp": int(pcm.numel() * 1000 / rate)}))
        writer.write(encode_event("ping", {"text": "end"}))         # answered in order: marks the end of the replies
        await writer.drain()
        while True:
            event = await asyncio.wait_for(read_event(reader), timeout=60)
            if event is None or event[0] == "pong":
                break
            if event[0] == "detection":
                hits.append(event[1])
    finally:
        writer.close()
    return hits
