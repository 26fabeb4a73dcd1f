"""Shared secret for authenticating launcher RPC messages.

Parity: horovod/runner/common/util/secret.py:26-36.
"""
import hashlib
import hmac
import os

SECRET_LENGTH = 32
DIGEST_LENGTH = 32
HOROVOD_SECRET_KEY = "_HOROVOD_SECRET_KEY"


def make_secret_key():
    return os.urandom(SECRET_LENGTH)


def compute_digest(key, message):
    return hmac.new(key, message, hashlib.sha256).digest()


def check_digest(key, message, digest):
    return hmac.compare_digest(compute_digest(key, message), digest)
