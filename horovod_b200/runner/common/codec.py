"""Objects as printable text: cloudpickle + base64, for values that travel in
command lines, environment variables and the HTTP key-value store.
Parity: horovod/runner/common/util/codec.py."""
import base64

import cloudpickle


def dumps_base64(obj, to_ascii=True):
    """Serialises ``obj``; a ``str`` by default, ``bytes`` with to_ascii=False."""
    encoded = base64.b64encode(cloudpickle.dumps(obj))
    return encoded.decode("ascii") if to_ascii else encoded


def loads_base64(encoded):
    """Inverse of dumps_base64; accepts str or bytes."""
    return cloudpickle.loads(base64.b64decode(encoded))
