"""Prometheus endpoint for a parameter server process.

``serve_metrics(server, port)`` starts a daemon HTTP thread that answers ``GET /metrics`` with the
server's per-request series (``ps_requests_total``, ``ps_errors_total``, ``ps_requests_size_bytes``,
``ps_response_size_bytes``, ``ps_request_duration_ms`` histogram, labelled with request type, storage id
and node id: the series of pico-ps/service/Service.cpp:23-33) plus storage gauges taken from
``Server.storage_size``. ``handler_metrics_text`` renders a handler's client-side counters
(``ps_wait_request_count``, ``ps_wait_duration_ms_sum``: pico-ps/handler/Handler.cpp:14-18).
"""
from __future__ import annotations

import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Iterable, Optional


def server_metrics_text(server, storage_ids: Optional[Iterable[int]] = None) -> str:
    text = server.metrics_text()
    if storage_ids:
        text += "# TYPE ps_storage_items gauge\n"
        for sid in storage_ids:
            text += f'ps_storage_items{{node_id="{server.node_id()}",storage_id="{sid}"}} {server.storage_size(sid)}\n'
    return text


def handler_metrics_text(handler, name: str) -> str:
    m = handler.metrics()
    lab = f'{{handler="{name}"}}'
    text = (f"ps_wait_request_count{lab} {m['requests']}\n"
            f"ps_wait_retry_count{lab} {m['retries']}\n"
            f"ps_wait_error_count{lab} {m['errors']}\n"
            f"ps_wait_duration_ms_sum{lab} {m['wait_us'] / 1e3}\n")
    if m.get("sends"):      # pull handlers: the request-building side (pico-ps/handler/PullHandler.cpp:11-15)
        text += (f"ps_pull_send_request_count{lab} {m['sends']}\n"
                 f"ps_pull_send_duration_ms_sum{lab} {m['send_us'] / 1e3}\n")
    return text


def serve_metrics(server, port: int = 0, storage_ids: Optional[Iterable[int]] = None, host: str = "127.0.0.1"):
    """Returns ``(http_server, port)``; call ``http_server.shutdown()`` to stop."""
    ids = list(storage_ids or [])

    class _H(BaseHTTPRequestHandler):
        def do_GET(self):  # noqa: N802
            if self.path.split("?")[0] != "/metrics":
                self.send_response(404)
                self.end_headers()
                return
            body = server_metrics_text(server, ids).encode()
            self.send_response(200)
            self.send_header("Content-Type", "text/plain; version=0.0.4")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def log_message(self, *a):  # keep the server's stderr clean
            pass

    httpd = ThreadingHTTPServer((host, port), _H)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    return httpd, httpd.server_address[1]
