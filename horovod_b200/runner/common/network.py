"""Minimal authenticated RPC used between the launcher, the elastic driver
and workers: length-prefixed cloudpickle messages over TCP, each carrying an
HMAC-SHA256 digest computed with a per-job secret. A service answers a
request object with a response object; a client tries all advertised
addresses of a service and keeps the ones that answer.

Parity: horovod/runner/common/util/network.py:56-306.
"""
import queue
import socket
import socketserver
import struct
import threading

import cloudpickle

from horovod_b200.runner.common import secret


class PingRequest:
    pass


class NoValidAddressesFound(Exception):
    pass


class PingResponse:
    def __init__(self, service_name, source_address):
        self.service_name = service_name
        self.source_address = source_address


class AckResponse:
    pass


class Wire:
    """Message framing: 4-byte length, 32-byte digest, pickled body."""

    def __init__(self, key):
        self._key = key

    def write(self, obj, wfile):
        message = cloudpickle.dumps(obj)
        digest = secret.compute_digest(self._key, message)
        wfile.write(struct.pack("i", len(message)))
        wfile.write(digest)
        wfile.write(message)
        wfile.flush()

    def read(self, rfile):
        header = rfile.read(4)
        if len(header) < 4:
            raise EOFError("connection closed")
        (length,) = struct.unpack("i", header)
        digest = rfile.read(secret.DIGEST_LENGTH)
        message = rfile.read(length)
        if not secret.check_digest(self._key, message, digest):
            raise Exception("Security error: digest did not match the message.")
        return cloudpickle.loads(message)


class BasicService:
    def __init__(self, service_name, key, nics=None):
        self._service_name = service_name
        self._wire = Wire(key)
        self._nics = nics
        self._server, _ = find_port(lambda addr: socketserver.ThreadingTCPServer(
            addr, self._make_handler()))
        self._server.daemon_threads = True
        self._port = self._server.socket.getsockname()[1]
        self._addresses = self._get_local_addresses()
        self._thread = threading.Thread(target=self._server.serve_forever, daemon=True,
                                        name="hvd-service-" + service_name)
        self._thread.start()

    def _make_handler(self):
        server = self

        class _Handler(socketserver.StreamRequestHandler):
            def handle(self):
                try:
                    req = server._wire.read(self.rfile)
                    resp = server._handle(req, self.client_address)
                    if resp is None:
                        raise Exception("Handler did not return a response.")
                    server._wire.write(resp, self.wfile)
                except (EOFError, ConnectionError):
                    pass
                except Exception:  # noqa: BLE001 - a bad message must not kill the service
                    pass
        return _Handler

    def _handle(self, req, client_address):
        if isinstance(req, PingRequest):
            return PingResponse(self._service_name, client_address[0])
        raise NotImplementedError(req)

    def _get_local_addresses(self):
        """{interface name: [(ipv4, port)]} for every interface that is up,
        filtered to ``nics`` when given (loopback is always kept last so a
        single-host job still works)."""
        result = {}
        try:
            import psutil
            for intf, addrs in psutil.net_if_addrs().items():
                if self._nics and intf not in self._nics:
                    continue
                for a in addrs:
                    if a.family == socket.AF_INET:
                        result.setdefault(intf, []).append((a.address, self._port))
        except Exception:  # noqa: BLE001 - psutil missing or unreadable: fall back below
            result = {}
        if not result:
            result = {"lo": [("127.0.0.1", self._port)]}
            try:
                host_ip = socket.gethostbyname(socket.gethostname())
                if host_ip != "127.0.0.1":
                    result["host"] = [(host_ip, self._port)]
            except OSError:
                pass
            if self._nics:
                result = {k: v for k, v in result.items() if k in self._nics} or result
        return result

    def addresses(self):
        return {k: list(v) for k, v in self._addresses.items()}

    def get_port(self):
        return self._port

    def shutdown(self):
        self._server.shutdown()
        self._server.server_close()
        self._thread.join(timeout=5)


class BasicClient:
    def __init__(self, service_name, addresses, key, verbose=0, match_intf=False,
                 probe_timeout=20, attempts=3):
        self._service_name = service_name
        self._wire = Wire(key)
        self._verbose = verbose
        self._match_intf = match_intf
        self._probe_timeout = probe_timeout
        self._attempts = attempts
        self._addresses = self._probe(addresses)
        if not self._addresses:
            raise NoValidAddressesFound(
                "horovodrun was unable to connect to %s on any of the following addresses: %s"
                % (service_name, addresses))

    def _probe(self, addresses):
        result_queue = queue.Queue()
        threads = []
        for intf, intf_addresses in addresses.items():
            for addr in intf_addresses:
                t = threading.Thread(target=self._probe_one, args=(intf, addr, result_queue),
                                     daemon=True)
                t.start()
                threads.append(t)
        for t in threads:
            t.join()
        result = {}
        while not result_queue.empty():
            intf, addr = result_queue.get()
            result.setdefault(intf, []).append(addr)
        return result

    def _probe_one(self, intf, addr, result_queue):
        for _ in range(self._attempts):
            try:
                sock = socket.create_connection(tuple(addr), timeout=self._probe_timeout)
                rfile, wfile = sock.makefile("rb"), sock.makefile("wb")
                try:
                    self._wire.write(PingRequest(), wfile)
                    resp = self._wire.read(rfile)
                    if resp.service_name == self._service_name:
                        result_queue.put((intf, addr))
                    return
                finally:
                    rfile.close()
                    wfile.close()
                    sock.close()
            except Exception:  # noqa: BLE001 - try again / give up on this address
                pass

    def _send_one(self, addr, req):
        last = None
        for _ in range(self._attempts):
            try:
                sock = socket.create_connection(tuple(addr), timeout=self._probe_timeout)
                rfile, wfile = sock.makefile("rb"), sock.makefile("wb")
                try:
                    self._wire.write(req, wfile)
                    return self._wire.read(rfile)
                finally:
                    rfile.close()
                    wfile.close()
                    sock.close()
            except Exception as e:  # noqa: BLE001
                last = e
        raise last

    def _send(self, req):
        for addrs in self._addresses.values():
            for addr in addrs:
                return self._send_one(addr, req)
        raise NoValidAddressesFound(self._service_name)

    def addresses(self):
        return self._addresses


def find_port(server_factory, start=1024 + 0, attempts=200):
    """Binds a server on an ephemeral port."""
    last = None
    for _ in range(attempts):
        try:
            server = server_factory(("0.0.0.0", 0))
            return server, server.socket.getsockname()[1]
        except OSError as e:
            last = e
    raise Exception("Unable to find a port to bind to: %s" % last)
