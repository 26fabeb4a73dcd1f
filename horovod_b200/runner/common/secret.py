"""The job's shared secret: the launcher draws it once, hands it to every
process it starts, and both ends of the launcher's RPC sign message bodies
with it (HMAC-SHA256), so that a service only acts on requests from its own
job.

Same role and names as horovod/runner/common/util/secret.py:26-36.
"""
import hashlib
import hmac
import secrets

_HASH = hashlib.sha256
SECRET_LENGTH = 32                      # bytes of key material
DIGEST_LENGTH = _HASH().digest_size     # bytes a signature occupies in a frame
HOROVOD_SECRET_KEY = "_HOROVOD_SECRET_KEY"  # environment variable carrying the encoded key


def make_secret_key():
    return secrets.token_bytes(SECRET_LENGTH)


def compute_digest(key, message):
    return hmac.digest(key, message, _HASH)


def check_digest(key, message, digest):
    """Constant-time comparison; a digest of the wrong length never matches."""
    expected = compute_digest(key, message)
    return len(digest) == len(expected) and hmac.compare_digest(expected, digest)
