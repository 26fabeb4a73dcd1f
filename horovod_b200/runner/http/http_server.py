"""Threaded HTTP key-value server used for rendezvous.

``PUT /scope/key`` stores a value, ``GET /scope/key`` returns it (404 while
absent), ``DELETE /scope/key`` counts one finished rank for the scope; when
every rank of a scope has finished, the scope's keys are dropped.
``RendezvousServer`` adds the slot table the launcher publishes so that
workers can look up their rank layout; the elastic driver plugs a handler in
for the ``rank_and_size`` and ``worker_addresses`` scopes.

Parity: horovod/runner/http/http_server.py:35-218.
"""
import collections
import socket
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

OK, BAD_REQUEST, NOT_FOUND, TIMEOUT = 200, 400, 404, 408

SINGLE_REQUEST_TIMEOUT = 600


def _split(path):
    parts = path.lstrip("/").split("/", 1)
    if len(parts) != 2 or not parts[0] or not parts[1]:
        return None, None
    return parts[0], parts[1]


class KVStoreHandler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.0"

    def log_message(self, fmt, *args):  # silence per-request logging
        pass

    def _reply(self, code, body=b""):
        self.send_response(code)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        if body:
            self.wfile.write(body)

    def do_GET(self):
        scope, key = _split(self.path)
        if scope is None:
            return self._reply(BAD_REQUEST)
        custom = self.server.custom_get(scope, key)
        if custom is not None:
            code, body = custom
            return self._reply(code, body)
        with self.server.cache_lock:
            value = self.server.cache.get(scope, {}).get(key)
        if value is None:
            return self._reply(NOT_FOUND)
        self._reply(OK, value)

    def do_PUT(self):
        scope, key = _split(self.path)
        if scope is None:
            return self._reply(BAD_REQUEST)
        length = int(self.headers.get("Content-Length", "0"))
        value = self.rfile.read(length) if length else b""
        if self.server.custom_put(scope, key, value):
            return self._reply(OK)
        with self.server.cache_lock:
            self.server.cache.setdefault(scope, {})[key] = value
        self._reply(OK)

    def do_DELETE(self):
        scope, key = _split(self.path)
        if scope is None:
            return self._reply(BAD_REQUEST)
        self.server.finish(scope, key)
        self._reply(OK)


class _Server(ThreadingHTTPServer):
    daemon_threads = True
    allow_reuse_address = True
    request_queue_size = 512

    def __init__(self, addr):
        super().__init__(addr, KVStoreHandler)
        self.cache_lock = threading.Lock()
        self.cache = {}
        self.finished = collections.defaultdict(set)
        self.scope_sizes = {}
        self.get_hook = None
        self.put_hook = None

    def custom_get(self, scope, key):
        return self.get_hook(scope, key) if self.get_hook else None

    def custom_put(self, scope, key, value):
        return self.put_hook(scope, key, value) if self.put_hook else False

    def finish(self, scope, key):
        with self.cache_lock:
            self.finished[scope].add(key)
            expected = self.scope_sizes.get(scope)
            if expected is not None and len(self.finished[scope]) >= expected:
                self.cache.pop(scope, None)
                self.finished.pop(scope, None)


class KVStoreServer:
    """Plain key-value server (also used by the programmatic run() API to
    carry the pickled function and the per-rank results)."""

    def __init__(self, verbose=0):
        self.verbose = verbose
        self.httpd = None
        self.thread = None
        self.port = None

    def start_server(self, port=0):
        self.httpd = _Server(("0.0.0.0", port))
        self.port = self.httpd.server_address[1]
        self.thread = threading.Thread(target=self.httpd.serve_forever, daemon=True,
                                       name="hvd-kv-server")
        self.thread.start()
        return self.port

    def shutdown_server(self):
        if self.httpd is not None:
            self.httpd.shutdown()
            self.httpd.server_close()
            self.httpd = None
        if self.thread is not None:
            self.thread.join(timeout=5)
            self.thread = None

    # direct access for the process that hosts the server
    def put(self, scope, key, value):
        with self.httpd.cache_lock:
            self.httpd.cache.setdefault(scope, {})[key] = value

    def get(self, scope, key):
        with self.httpd.cache_lock:
            return self.httpd.cache.get(scope, {}).get(key)


class RendezvousServer(KVStoreServer):
    """KV server that also knows the job's slot assignment."""

    def __init__(self, verbose=0):
        super().__init__(verbose)
        self.host_assignments = None

    def start(self, handler_cls=None, port=0):
        port = self.start_server(port)
        return port

    def init(self, host_alloc_plan):
        """Publishes a (new) slot plan: list of SlotInfo. Clears the keys of
        earlier rounds so stale addresses cannot be picked up."""
        self.host_assignments = host_alloc_plan
        with self.httpd.cache_lock:
            self.httpd.cache.clear()
            self.httpd.finished.clear()
            size = len(host_alloc_plan)
            self.httpd.scope_sizes = {"global": size}

    def set_hooks(self, get_hook=None, put_hook=None):
        self.httpd.get_hook = get_hook
        self.httpd.put_hook = put_hook

    def stop(self):
        self.shutdown_server()


def local_ip_for(host="8.8.8.8"):
    """Best-effort address of this machine as seen from ``host``."""
    try:
        s = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        s.connect((host, 80))
        ip = s.getsockname()[0]
        s.close()
        return ip
    except OSError:
        return "127.0.0.1"
