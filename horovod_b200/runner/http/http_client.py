"""Python objects in the launcher's HTTP key-value store (the rendezvous
server): values are stored pickled and base64-encoded under /scope/key.
Parity: horovod/runner/http/http_client.py."""
from urllib.error import HTTPError, URLError
from urllib.request import Request, urlopen

from horovod_b200.runner.common import codec


def _url(addr, port, scope, key):
    return "http://%s:%s/%s/%s" % (addr, port, scope, key)


def read_data_from_kvstore(addr, port, scope, key):
    try:
        with urlopen(Request(_url(addr, port, scope, key))) as response:
            return codec.loads_base64(response.read())
    except (HTTPError, URLError) as e:
        raise RuntimeError("Read data from KVStore server failed.", e)


def put_data_into_kvstore(addr, port, scope, key, value):
    try:
        request = Request(_url(addr, port, scope, key),
                          data=codec.dumps_base64(value, to_ascii=False), method="PUT")
        with urlopen(request):
            pass
    except (HTTPError, URLError) as e:
        raise RuntimeError("Put data input KVStore server failed.", e)
