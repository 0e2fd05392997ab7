"""Data-parallel front end for several API servers.

Routes every request to the replica with the fewest requests in flight and, while any
replica is busy, keeps the idle ones stepping with one-token keep-alive requests marked
``extra_args: {"is_idle": true}`` so that expert-parallel collectives that span the replicas
never wait for a rank that has nothing to do (benchmarks/router.py:16-168 of the reference).
``/start_profile`` and ``/stop_profile`` go to replica 0 only.

Example: python benchmarks/router.py --port 9000 --backends 127.0.0.1:8000 127.0.0.1:8001
"""
import argparse
import asyncio
import json


class Router:
    def __init__(self, backends, idle_interval=0.02):
        self.backends = list(backends)
        self.active = [0] * len(self.backends)
        self.idle_interval = idle_interval
        self.session = None
        self._pump_task = None

    def pick(self) -> int:
        return min(range(len(self.backends)), key=lambda i: self.active[i])

    async def _session(self):
        import aiohttp
        if self.session is None:
            self.session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=6 * 3600))
        return self.session

    async def _idle_pump(self):
        """While at least one replica works, the others receive keep-alive requests."""
        body = {"prompt": [1], "max_tokens": 1, "temperature": 0.0,
                "extra_args": {"is_idle": True}}
        while True:
            await asyncio.sleep(self.idle_interval)
            if not any(self.active):
                continue
            s = await self._session()
            for i, n in enumerate(self.active):
                if n == 0:
                    try:
                        async with s.post(f"http://{self.backends[i]}/v1/completions",
                                          json=body) as r:
                            await r.read()
                    except Exception:  # noqa: BLE001
                        pass

    def app(self):
        from fastapi import FastAPI, Request
        from fastapi.responses import Response, StreamingResponse
        app = FastAPI()
        router = self

        @app.on_event("startup")
        async def _start():
            if len(router.backends) > 1:
                router._pump_task = asyncio.create_task(router._idle_pump())

        async def forward(path: str, request: Request, idx: int):
            s = await router._session()
            body = await request.body()
            router.active[idx] += 1
            try:
                resp = await s.post(f"http://{router.backends[idx]}{path}", data=body,
                                    headers={"content-type": "application/json"})
            except Exception:
                router.active[idx] -= 1
                raise

            async def stream():
                try:
                    async for chunk in resp.content.iter_any():
                        yield chunk
                finally:
                    router.active[idx] -= 1
                    resp.release()
            return StreamingResponse(stream(), status_code=resp.status,
                                     media_type=resp.headers.get("content-type"))

        @app.post("/v1/completions")
        async def completions(request: Request):
            return await forward("/v1/completions", request, router.pick())

        @app.post("/start_profile")
        async def start_profile(request: Request):
            return await forward("/start_profile", request, 0)

        @app.post("/stop_profile")
        async def stop_profile(request: Request):
            return await forward("/stop_profile", request, 0)

        @app.get("/health")
        async def health():
            return {"status": "ok", "active": router.active}

        return app


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=9000)
    ap.add_argument("--backends", nargs="+", required=True)
    a = ap.parse_args()
    import uvicorn
    uvicorn.run(Router(a.backends).app(), host=a.host, port=a.port, log_level="warning")


if __name__ == "__main__":
    main()
