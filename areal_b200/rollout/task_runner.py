"""Background asyncio runner: a thread owning an event loop that executes submitted
coroutines and hands results back through a thread-safe queue.

Role of the reference's ``areal/infra/async_task_runner.py:73-415`` (uvloop thread, input /
output queues, pause / resume, fail-fast exception propagation).
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Any, Awaitable, Callable, Optional


class TaskQueueFullError(RuntimeError):
    pass


@dataclass
class TaskResult:
    task_id: int
    data: Any
    create_time: float
    error: Optional[BaseException] = None


class AsyncTaskRunner:
    def __init__(self, max_queue_size: int = 4096, poll_sleep: float = 0.005, name: str = "rollout-runner"):
        self._in: "queue.Queue[tuple[int, Callable[[], Awaitable[Any]], float]]" = queue.Queue(maxsize=max_queue_size)
        self._out: "queue.Queue[TaskResult]" = queue.Queue()
        self._paused = threading.Event()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._loop: Optional[asyncio.AbstractEventLoop] = None
        self._exc: Optional[BaseException] = None
        self._exc_tb: str = ""
        self._next_id = 0
        self._id_lock = threading.Lock()
        self._poll = poll_sleep
        self._name = name
        self._running = 0
        self._shutdown_hooks: list[Callable[[], Awaitable[None]]] = []

    # ------------------------------------------------------------------ lifecycle
    def initialize(self):
        if self._thread is not None:
            return
        self._thread = threading.Thread(target=self._thread_main, name=self._name, daemon=True)
        self._thread.start()

    def destroy(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None

    def register_shutdown_hook(self, fn):
        self._shutdown_hooks.append(fn)

    def _thread_main(self):
        try:
            try:
                import uvloop

                loop = uvloop.new_event_loop()
            except Exception:
                loop = asyncio.new_event_loop()
            asyncio.set_event_loop(loop)
            self._loop = loop
            loop.run_until_complete(self._main())
        except BaseException as e:  # propagate to the caller thread
            self._exc, self._exc_tb = e, traceback.format_exc()
        finally:
            try:
                if self._loop is not None:
                    self._loop.close()
            except Exception:
                pass

    async def _main(self):
        pending: set[asyncio.Task] = set()
        try:
            while not self._stop.is_set():
                while not self._paused.is_set():
                    try:
                        tid, factory, t0 = self._in.get_nowait()
                    except queue.Empty:
                        break
                    task = asyncio.ensure_future(self._run_one(tid, factory, t0))
                    pending.add(task)
                    self._running += 1
                if pending:
                    done, pending = await asyncio.wait(pending, timeout=0.05, return_when=asyncio.FIRST_COMPLETED)
                    for d in done:
                        self._running -= 1
                        d.result()
                else:
                    await asyncio.sleep(self._poll)
        finally:
            for t in pending:
                t.cancel()
            if pending:
                await asyncio.gather(*pending, return_exceptions=True)
            for hook in self._shutdown_hooks:
                try:
                    await hook()
                except Exception:
                    pass

    async def _run_one(self, tid, factory, t0):
        try:
            res = await factory()
            self._out.put(TaskResult(tid, res, t0))
        except asyncio.CancelledError:
            raise
        except BaseException as e:
            self._out.put(TaskResult(tid, None, t0, error=e))

    # ------------------------------------------------------------------ API
    def check_health(self):
        if self._exc is not None:
            raise RuntimeError(f"rollout runner thread died:\n{self._exc_tb}") from self._exc

    def new_task_id(self) -> int:
        with self._id_lock:
            self._next_id += 1
            return self._next_id

    def submit(self, coro_factory: Callable[[], Awaitable[Any]], task_id: Optional[int] = None) -> int:
        self.check_health()
        tid = task_id if task_id is not None else self.new_task_id()
        try:
            self._in.put_nowait((tid, coro_factory, time.monotonic()))
        except queue.Full as e:
            raise TaskQueueFullError("rollout input queue is full") from e
        return tid

    def poll(self, timeout: float = 0.05) -> Optional[TaskResult]:
        self.check_health()
        try:
            return self._out.get(timeout=timeout)
        except queue.Empty:
            return None

    def pause(self):
        self._paused.set()

    def resume(self):
        self._paused.clear()

    def is_paused(self) -> bool:
        return self._paused.is_set()

    def input_queue_size(self) -> int:
        return self._in.qsize()

    def output_queue_size(self) -> int:
        return self._out.qsize()

    @property
    def running(self) -> int:
        return self._running
