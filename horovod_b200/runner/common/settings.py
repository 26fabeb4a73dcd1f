"""Launcher settings passed around between the CLI, the drivers and the
process launchers.

Parity: horovod/runner/common/util/settings.py.
"""


class BaseSettings:
    def __init__(self, num_proc=None, verbose=0, ssh_port=None, ssh_identity_file=None,
                 extra_mpi_args=None, tcp_flag=None, binding_args=None, key=None,
                 start_timeout=None, output_filename=None, run_func_mode=None,
                 nics=None, elastic=False, prefix_output_with_timestamp=False):
        self.num_proc = num_proc
        self.verbose = verbose
        self.ssh_port = ssh_port
        self.ssh_identity_file = ssh_identity_file
        self.extra_mpi_args = extra_mpi_args
        self.tcp_flag = tcp_flag
        self.binding_args = binding_args
        self.key = key
        self.start_timeout = start_timeout
        self.output_filename = output_filename
        self.run_func_mode = run_func_mode
        self.nics = nics
        self.elastic = elastic
        self.prefix_output_with_timestamp = prefix_output_with_timestamp


class Settings(BaseSettings):
    def __init__(self, hosts=None, **kwargs):
        super().__init__(**kwargs)
        self.hosts = hosts


class ElasticSettings(BaseSettings):
    def __init__(self, discovery=None, min_np=None, max_np=None, elastic_timeout=None,
                 reset_limit=None, cooldown_range=None, **kwargs):
        kwargs["elastic"] = True
        super().__init__(**kwargs)
        self.discovery = discovery
        self.min_np = min_np
        self.max_np = max_np
        self.elastic_timeout = elastic_timeout
        self.reset_limit = reset_limit
        self.cooldown_range = cooldown_range
