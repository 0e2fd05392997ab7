"""Prefill / decode disaggregation proxy (1P1D or xPyD, round robin).

Clients talk to this proxy; for every completion request it first sends the prompt to a
prefill server with ``max_tokens = 1`` and ``kv_transfer_params = {"do_remote_decode": True,
"remote": <decode server's KV address>}``, then forwards the original request to a decode
server with ``{"do_remote_prefill": True, "remote": <prefill KV address>,
"remote_request_id": <id of the prefill request>}`` and relays its answer.  Servers register
themselves by listing ``http_address=kv_address`` pairs on the command line (the reference's
xPyD proxy learns them over a ZMQ registration socket,
benchmarks/disagg_benchmarks/disagg_proxy_p2p_nccl_xpyd.py:22-40).

  python benchmarks/disagg_benchmarks/disagg_proxy.py --port 8000 \
      --prefill 127.0.0.1:8100=127.0.0.1:21001 --decode 127.0.0.1:8200=127.0.0.1:22001
"""
import argparse
import itertools
import json
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from urllib import request as urlreq


def _post(addr: str, path: str, body: dict, timeout: float = 600.0) -> dict:
    req = urlreq.Request(f"http://{addr}{path}", data=json.dumps(body).encode(),
                         headers={"Content-Type": "application/json"})
    with urlreq.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


class Proxy:
    def __init__(self, prefill: list, decode: list):
        self.prefill = itertools.cycle(prefill)      # (http, kv) pairs
        self.decode = itertools.cycle(decode)

    def handle(self, path: str, body: dict) -> dict:
        p_http, p_kv = next(self.prefill)
        d_http, d_kv = next(self.decode)
        rid = "disagg-" + uuid.uuid4().hex[:12]
        first = dict(body, max_tokens=1, stream=False, request_id=rid,
                     kv_transfer_params={"do_remote_decode": True, "remote": d_kv})
        _post(p_http, path, first)
        second = dict(body, kv_transfer_params={"do_remote_prefill": True, "remote": p_kv,
                                                "remote_request_id": rid})
        return _post(d_http, path, second)


def _pairs(items):
    out = []
    for it in items:
        http, _, kv = it.partition("=")
        out.append((http, kv or http))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--prefill", action="append", required=True)
    ap.add_argument("--decode", action="append", required=True)
    a = ap.parse_args()
    proxy = Proxy(_pairs(a.prefill), _pairs(a.decode))

    class H(BaseHTTPRequestHandler):
        def do_POST(self):
            n = int(self.headers.get("Content-Length", "0"))
            body = json.loads(self.rfile.read(n) or b"{}")
            try:
                out, code = proxy.handle(self.path, body), 200
            except Exception as e:          # noqa: BLE001 - reported to the client
                out, code = {"error": str(e)}, 502
            data = json.dumps(out).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def log_message(self, *args):
            pass

    ThreadingHTTPServer(("0.0.0.0", a.port), H).serve_forever()


if __name__ == "__main__":
    main()
