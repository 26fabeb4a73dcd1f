"""Minimal authenticated RPC used between the launcher, the elastic driver
and workers. One request and one response per TCP connection; each message is
a frame of a fixed header (body length and HMAC-SHA256 of the body, keyed with
the job's secret) followed by the cloudpickled object. A service answers a
request object with a response object; a client learns at construction which
of a service's advertised addresses reach it and uses those afterwards.

What callers rely on (and what horovod/runner/common/util/network.py:56-306
offers its callers): ``BasicService`` with an overridable ``_handle``,
``addresses()``, ``get_port()``, ``shutdown()``; ``BasicClient`` with
``_send(request)`` and ``addresses()``; ``PingRequest`` / ``PingResponse`` /
``AckResponse``; ``NoValidAddressesFound``; ``find_port``.
"""
import concurrent.futures
import contextlib
import socket
import socketserver
import struct
import threading

import cloudpickle

from horovod_b200.runner.common import secret


class PingRequest:
    """Answered by every service with its name and the caller's address."""


class PingResponse:
    def __init__(self, service_name, source_address):
        self.service_name = service_name
        self.source_address = source_address


class AckResponse:
    """The answer of requests that have nothing to return."""


class NoValidAddressesFound(Exception):
    pass


class Wire:
    """Frames: ``!I`` body length, then the digest, then the body."""

    _LENGTH = struct.Struct("!I")

    def __init__(self, key):
        self._key = key

    def write(self, obj, wfile):
        body = cloudpickle.dumps(obj)
        wfile.write(self._LENGTH.pack(len(body)) + secret.compute_digest(self._key, body) + body)
        wfile.flush()

    def read(self, rfile):
        head = rfile.read(self._LENGTH.size + secret.DIGEST_LENGTH)
        if len(head) < self._LENGTH.size + secret.DIGEST_LENGTH:
            raise EOFError("connection closed")
        (length,) = self._LENGTH.unpack_from(head)
        body = rfile.read(length)
        if len(body) < length:
            raise EOFError("connection closed inside a message")
        if not secret.check_digest(self._key, body, head[self._LENGTH.size:]):
            raise Exception("Security error: digest did not match the message.")
        return cloudpickle.loads(body)


def _ipv4_by_interface(port, nics=None):
    """{interface: [(address, port)]} of this machine, restricted to ``nics``
    when given; at least the loopback (and the host name's address) when the
    interfaces cannot be listed."""
    found = {}
    try:
        import psutil
        for name, infos in psutil.net_if_addrs().items():
            if nics and name not in nics:
                continue
            ips = [(i.address, port) for i in infos if i.family == socket.AF_INET]
            if ips:
                found[name] = ips
    except Exception:  # noqa: BLE001 - psutil missing or unreadable
        found = {}
    if found:
        return found
    fallback = {"lo": [("127.0.0.1", port)]}
    with contextlib.suppress(OSError):
        host_ip = socket.gethostbyname(socket.gethostname())
        if host_ip != "127.0.0.1":
            fallback["host"] = [(host_ip, port)]
    if nics:
        wanted = {k: v for k, v in fallback.items() if k in nics}
        return wanted or fallback
    return fallback


class BasicService:
    """A threaded TCP server that reads one request per connection, passes it
    to ``_handle`` and writes back what that returns. Subclasses extend
    ``_handle`` and call the base for requests they do not know."""

    def __init__(self, service_name, key, nics=None):
        self._service_name = service_name
        self._wire = Wire(key)
        self._nics = nics
        service = self

        class Connection(socketserver.StreamRequestHandler):
            def handle(self):
                # A bad or truncated message ends this connection, never the service.
                with contextlib.suppress(Exception):
                    request = service._wire.read(self.rfile)
                    response = service._handle(request, self.client_address)
                    if response is None:
                        raise Exception("Handler did not return a response.")
                    service._wire.write(response, self.wfile)

        self._server, self._port = find_port(
            lambda address: socketserver.ThreadingTCPServer(address, Connection))
        self._server.daemon_threads = True
        self._addresses = _ipv4_by_interface(self._port, nics)
        self._thread = threading.Thread(target=self._server.serve_forever, daemon=True,
                                        name="hvd-service-" + service_name)
        self._thread.start()

    def _handle(self, req, client_address):
        if isinstance(req, PingRequest):
            return PingResponse(self._service_name, client_address[0])
        raise NotImplementedError(req)

    def addresses(self):
        return {name: list(pairs) for name, pairs in self._addresses.items()}

    def get_port(self):
        return self._port

    def shutdown(self):
        self._server.shutdown()
        self._server.server_close()
        self._thread.join(timeout=5)


class BasicClient:
    """Talks to one service. ``addresses`` is the service's
    ``{interface: [(ip, port)]}``; the constructor pings all of them at once
    and keeps those that answer with the right service name."""

    def __init__(self, service_name, addresses, key, verbose=0, match_intf=False,
                 probe_timeout=20, attempts=3):
        self._service_name = service_name
        self._wire = Wire(key)
        self._verbose = verbose
        self._match_intf = match_intf
        self._probe_timeout = probe_timeout
        self._attempts = attempts
        self._addresses = self._reachable(addresses)
        if not self._addresses:
            raise NoValidAddressesFound(
                "horovodrun was unable to connect to %s on any of the following addresses: %s"
                % (service_name, addresses))

    def _exchange(self, address, request):
        """One connection: send ``request``, return the response."""
        with socket.create_connection(tuple(address), timeout=self._probe_timeout) as sock:
            with sock.makefile("rb") as rfile, sock.makefile("wb") as wfile:
                self._wire.write(request, wfile)
                return self._wire.read(rfile)

    def _with_retries(self, address, request):
        error = None
        for _ in range(self._attempts):
            try:
                return self._exchange(address, request)
            except Exception as e:  # noqa: BLE001 - refused, reset, bad digest: try again
                error = e
        raise error

    def _answers(self, address):
        try:
            reply = self._with_retries(address, PingRequest())
        except Exception:  # noqa: BLE001 - unreachable from here
            return False
        return getattr(reply, "service_name", None) == self._service_name

    def _reachable(self, addresses):
        candidates = [(name, pair) for name, pairs in addresses.items() for pair in pairs]
        if not candidates:
            return {}
        with concurrent.futures.ThreadPoolExecutor(max_workers=len(candidates)) as pool:
            verdicts = list(pool.map(lambda c: self._answers(c[1]), candidates))
        kept = {}
        for (name, pair), ok in zip(candidates, verdicts):
            if ok:
                kept.setdefault(name, []).append(pair)
        return kept

    def _send(self, req):
        for pairs in self._addresses.values():
            for pair in pairs:
                return self._with_retries(pair, req)
        raise NoValidAddressesFound(self._service_name)

    def addresses(self):
        return self._addresses


def find_port(server_factory, attempts=200):
    """Lets the operating system pick a free port for the server that
    ``server_factory((host, port))`` creates; returns (server, port)."""
    error = None
    for _ in range(attempts):
        try:
            server = server_factory(("0.0.0.0", 0))
            return server, server.socket.getsockname()[1]
        except OSError as e:
            error = e
    raise Exception("Unable to find a port to bind to: %s" % error)
