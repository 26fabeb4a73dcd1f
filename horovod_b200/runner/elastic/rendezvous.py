"""Elastic additions to the rendezvous server: a worker asks for its place
with ``GET /rank_and_size/<host>:<local_rank>`` (which blocks until every
live worker of the round has asked), and announces its notification service
with ``PUT /worker_addresses/<host>:<local_rank>``.

Parity: horovod/runner/elastic/rendezvous.py:28-55.
"""
import pickle

from horovod_b200.runner.http.http_server import OK, BAD_REQUEST

GET_RANK_AND_SIZE = "rank_and_size"
PUT_WORKER_ADDRESSES = "worker_addresses"


def attach_elastic_rendezvous(server, driver):
    def on_get(scope, key):
        if scope != GET_RANK_AND_SIZE:
            return None
        try:
            host, local_rank = key.rsplit(":", 1)
            local_rank = int(local_rank)
        except ValueError:
            return BAD_REQUEST, b""
        driver.record_ready(host, local_rank)
        slot_info = driver.get_slot_info(host, local_rank)
        reply = "%s,%d" % (slot_info.to_response_string(), driver.rendezvous_round())
        return OK, reply.encode("ascii")

    def on_put(scope, key, value):
        if scope != PUT_WORKER_ADDRESSES:
            return False
        host, local_rank = key.rsplit(":", 1)
        addresses, secret_key = pickle.loads(value)
        driver.register_worker_server(host, int(local_rank), addresses, secret_key)
        return True

    server.set_hooks(get_hook=on_get, put_hook=on_put)
