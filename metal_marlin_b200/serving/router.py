"""Data-parallel front end: one HTTP endpoint in front of N replica servers.

Every replica is a complete server of this package (``serving/server.py``) on its own GPU; the router forwards each
request to the replica with the fewest requests in flight (ties: round robin), streams server-sent events through
unchanged, skips replicas whose ``/health`` fails until they answer again, and merges ``/metrics``.  Started by
``metal-marlin serve --dp N`` under ``torchrun`` (rank r serves on ``port + 1 + r``, rank 0 also runs the router on
``port``), or stand-alone with :func:`run_router` for replicas on other hosts.

Parity: the reference serves from one process and has no replica routing; its request-level load metrics
(``metal_marlin/serving/metrics.py``) are what the least-loaded choice uses here.
"""
from __future__ import annotations

import asyncio
import itertools
import time
from typing import Dict, List, Optional

import aiohttp
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, Response, StreamingResponse


class ReplicaRouter:
    def __init__(self, backends: List[str], health_interval_s: float = 2.0, timeout_s: float = 600.0):
        if not backends:
            raise ValueError("at least one backend")
        self.backends = [b.rstrip("/") for b in backends]
        self.inflight = [0] * len(backends)
        self.served = [0] * len(backends)
        self.healthy = [True] * len(backends)
        self._last_check = [0.0] * len(backends)
        self.health_interval_s, self.timeout_s = health_interval_s, timeout_s
        self._rr = itertools.count()
        self._session: Optional[aiohttp.ClientSession] = None

    async def session(self) -> aiohttp.ClientSession:
        if self._session is None or self._session.closed:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout_s))
        return self._session

    async def close(self) -> None:
        if self._session is not None and not self._session.closed:
            await self._session.close()

    def pick(self) -> int:
        """Healthy replica with the fewest requests in flight; equal loads rotate."""
        cand = [i for i, ok in enumerate(self.healthy) if ok] or list(range(len(self.backends)))
        low = min(self.inflight[i] for i in cand)
        best = [i for i in cand if self.inflight[i] == low]
        return best[next(self._rr) % len(best)]

    async def refresh_health(self, force: bool = False) -> None:
        now = time.monotonic()
        s = await self.session()
        for i, b in enumerate(self.backends):
            if not force and (self.healthy[i] or now - self._last_check[i] < self.health_interval_s):
                continue
            self._last_check[i] = now
            try:
                async with s.get(b + "/health", timeout=aiohttp.ClientTimeout(total=2.0)) as r:
                    self.healthy[i] = r.status == 200
            except Exception:
                self.healthy[i] = False

    async def forward(self, request: Request) -> Response:
        await self.refresh_health()
        body = await request.body()
        headers = {k: v for k, v in request.headers.items() if k.lower() in ("content-type", "authorization", "accept")}
        last_err = None
        for _ in range(len(self.backends)):
            i = self.pick()
            url = self.backends[i] + request.url.path + (("?" + request.url.query) if request.url.query else "")
            self.inflight[i] += 1
            try:
                s = await self.session()
                resp = await s.request(request.method, url, data=body if body else None, headers=headers)
            except Exception as e:          # replica gone: mark it and try the next one
                self.inflight[i] -= 1
                self.healthy[i] = False
                last_err = e
                continue
            self.served[i] += 1
            ctype = resp.headers.get("content-type", "application/json")
            if ctype.startswith("text/event-stream"):
                async def stream(resp=resp, i=i):
                    try:
                        async for chunk in resp.content.iter_any():
                            yield chunk
                    finally:
                        resp.release()
                        self.inflight[i] -= 1
                return StreamingResponse(stream(), status_code=resp.status, media_type="text/event-stream",
                                         headers={"x-mmb200-replica": str(i)})
            try:
                data = await resp.read()
            finally:
                resp.release()
                self.inflight[i] -= 1
            return Response(content=data, status_code=resp.status, media_type=ctype, headers={"x-mmb200-replica": str(i)})
        return JSONResponse(status_code=503, content={"error": {"message": f"no replica reachable: {last_err!r}",
                                                                "type": "service_unavailable", "code": "no_replica"}})

    def stats(self) -> Dict[str, list]:
        return {"backends": self.backends, "inflight": list(self.inflight), "served": list(self.served), "healthy": list(self.healthy)}


def make_app(router: ReplicaRouter) -> FastAPI:
    app = FastAPI(title="metal-marlin (B200) replica router", version="0.1.0")

    @app.get("/health")
    async def health():
        await router.refresh_health(force=True)
        return {"status": "ok" if any(router.healthy) else "degraded", "replicas": router.stats()}

    @app.get("/router/stats")
    async def stats():
        return router.stats()

    @app.get("/metrics")
    async def metrics():
        s = await router.session()
        parts = []
        for i, b in enumerate(router.backends):
            try:
                async with s.get(b + "/metrics", timeout=aiohttp.ClientTimeout(total=5.0)) as r:
                    text = await r.text()
                parts.append(f"# replica {i} ({b})\n" + text)
            except Exception:
                router.healthy[i] = False
        head = "".join(f'mmb200_router_inflight{{replica="{i}"}} {n}\nmmb200_router_served{{replica="{i}"}} {router.served[i]}\n'
                       for i, n in enumerate(router.inflight))
        return PlainTextResponse(head + "\n".join(parts), media_type="text/plain; version=0.0.4")

    @app.api_route("/v1/{path:path}", methods=["GET", "POST"])
    async def v1(path: str, request: Request):
        return await router.forward(request)

    return app


def run_router(backends: List[str], host: str = "127.0.0.1", port: int = 8000, log_level: str = "info") -> None:
    import uvicorn
    router = ReplicaRouter(backends)
    try:
        uvicorn.run(make_app(router), host=host, port=port, log_level=log_level)
    finally:
        try:
            asyncio.run(router.close())
        except Exception:
            pass
