"""Async façade over the :class:`LLM` for the HTTP layer: admission control, request streaming,
cancellation on client disconnect.

Parity: ``tensorrt_edgellm/server/runtime/engine_client.py`` (``EngineClient``,
``_AdmissionController`` — bounded queue → 429, queue timeout → 503, ``_IFBAdmissionGate``)."""
from __future__ import annotations

import asyncio
import threading
import time
from dataclasses import dataclass
from typing import AsyncIterator, List, Optional, Sequence, Tuple

from ..runtime.llm import LLM, RequestOutput
from ..runtime.runner import SamplingParams


class QueueFull(Exception):
    """More requests are waiting than ``max_queued_requests`` allows (HTTP 429)."""


class QueueTimeout(Exception):
    """The request waited longer than ``queue_timeout`` for a slot (HTTP 503)."""


class EngineUnavailable(Exception):
    """The engine stopped accepting work, e.g. after repeated session failures (HTTP 503)."""


class AdmissionController:
    """Bounds the number of requests in the server at once.  ``slots`` requests run, up to
    ``max_queued`` wait; a waiter that is not admitted within ``timeout_s`` gives up."""

    def __init__(self, slots: int, max_queued: int, timeout_s: float):
        self.slots, self.max_queued, self.timeout_s = slots, max_queued, timeout_s
        self._running = 0
        self._waiting = 0
        self._cv = threading.Condition()

    def acquire(self) -> None:
        with self._cv:
            if self._running < self.slots and self._waiting == 0:
                self._running += 1
                return
            if self._waiting >= self.max_queued:
                raise QueueFull(f"{self._waiting} requests already queued")
            self._waiting += 1
            deadline = time.monotonic() + self.timeout_s
            try:
                while self._running >= self.slots:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        raise QueueTimeout(f"no slot within {self.timeout_s:.0f} s")
                    self._cv.wait(left)
                self._running += 1
            finally:
                self._waiting -= 1

    def release(self) -> None:
        with self._cv:
            self._running -= 1
            self._cv.notify()

    @property
    def depth(self) -> Tuple[int, int]:
        with self._cv:
            return self._running, self._waiting


@dataclass
class StreamDelta:
    token_ids: List[int]
    text: str
    finished: bool
    finish_reason: Optional[str] = None


class EngineClient:
    def __init__(self, llm: LLM, max_queued_requests: int = 256, queue_timeout: float = 600.0):
        self.llm = llm
        # With in-flight batching the native engine queues by itself, the gate only bounds the backlog;
        # without it, one static batch runs at a time.
        slots = llm.max_batch_size * 4 if llm.engine is not None else 1
        self.admission = AdmissionController(slots, max_queued_requests, queue_timeout)
        self._lock = threading.Lock()          # serialises static-batch generation

    def ready(self) -> Tuple[bool, str]:
        if self.llm.engine is not None:
            st = self.llm.engine.status()
            return bool(st.available), st.unavailable_reason
        return True, ""

    # ---- blocking bodies run in worker threads ------------------------------------------------------
    def _generate_blocking(self, ids: Sequence[int], sp: SamplingParams, priority: int) -> RequestOutput:
        self.admission.acquire()
        try:
            ok, why = self.ready()
            if not ok:
                raise EngineUnavailable(why)
            prompt = ids if hasattr(ids, "embeds") else list(ids)         # a prepared multimodal prompt passes through
            if self.llm.engine is not None:
                return self.llm.generate([prompt], sp)[0]
            with self._lock:
                return self.llm.generate([prompt], sp)[0]
        finally:
            self.admission.release()

    async def generate_guided(self, ids: Sequence[int], sp: SamplingParams, guided, priority: int = 0) -> RequestOutput:
        """Constrained request: the constraint rides on the sampling parameters, so it batches like any other request."""
        import dataclasses
        return await self.generate(ids, dataclasses.replace(sp, guided=guided), priority)

    async def generate(self, ids: Sequence[int], sp: SamplingParams, priority: int = 0) -> RequestOutput:
        return await asyncio.get_running_loop().run_in_executor(None, self._generate_blocking, ids, sp, priority)

    async def stream(self, ids: Sequence[int], sp: SamplingParams, priority: int = 0) -> AsyncIterator[StreamDelta]:
        """Token deltas as they are produced.  Without the request engine the whole answer arrives as one delta."""
        loop = asyncio.get_running_loop()
        if self.llm.engine is None:
            out = await self.generate(ids, sp, priority)
            yield StreamDelta(out.token_ids, out.text or "", True, out.finish_reason)
            return
        await loop.run_in_executor(None, self.admission.acquire)
        q: asyncio.Queue = asyncio.Queue()
        cancelled = threading.Event()

        def pump():
            try:
                ok, why = self.ready()
                if not ok:
                    raise EngineUnavailable(why)
                handle = self.llm.submit(ids if hasattr(ids, "embeds") else list(ids), sp, priority)
                ch = handle.stream()
                pending = b""
                tok = self.llm.tokenizer
                while True:
                    if cancelled.is_set():
                        handle.cancel()
                    c = ch.wait_pop(0.25)
                    if c is None:
                        continue
                    text = ""
                    if tok is not None and hasattr(tok, "id_to_bytes"):
                        for t in c.token_ids:
                            pending += bytes(tok.id_to_bytes(t))
                        n = self.llm._rt.utf8_complete_prefix(pending)
                        text, pending = pending[:n].decode("utf-8", "replace"), pending[n:]
                    elif tok is not None:
                        text = tok.decode(c.token_ids)
                    reason = None
                    if c.finished:
                        rt = self.llm._rt
                        reason = {rt.FinishReason.Length: "length", rt.FinishReason.EndId: "stop", rt.FinishReason.StopWords: "stop",
                                  rt.FinishReason.Cancelled: "cancelled", rt.FinishReason.Error: "error"}.get(handle.reason(), "length")
                    loop.call_soon_threadsafe(q.put_nowait, StreamDelta(list(c.token_ids), text, bool(c.finished), reason))
                    if c.finished:
                        return
            except Exception as e:           # surfaced to the consumer, never lost in the thread
                loop.call_soon_threadsafe(q.put_nowait, e)
            finally:
                self.admission.release()

        threading.Thread(target=pump, daemon=True).start()
        try:
            while True:
                item = await q.get()
                if isinstance(item, Exception):
                    raise item
                yield item
                if item.finished:
                    return
        finally:
            cancelled.set()                  # client went away: the pump cancels the request
