"""``horovodrun``: command-line launcher.

    horovodrun -np 8 python train.py
    horovodrun -np 16 -H host1:8,host2:8 python train.py
    horovodrun -np 8 --min-np 4 --host-discovery-script ./discover.sh python train.py

Every tuning flag is turned into a HOROVOD_* environment variable for the
workers; a YAML ``--config-file`` supplies defaults that explicit flags
override.

Parity: horovod/runner/launch.py:58-770.
"""
import argparse
import os
import sys
import textwrap

import yaml

import horovod_b200
from horovod_b200.runner.common import config_parser, hosts as hosts_mod
from horovod_b200.runner.common.settings import ElasticSettings, Settings
from horovod_b200.runner.common.timeout import Timeout
from horovod_b200.runner import gloo_run as gloo
from horovod_b200.runner.util import cache as cache_mod

CACHE_FOLDER = os.path.join(os.path.expanduser("~"), ".horovod_b200")
CACHE_STALENESS_THRESHOLD_MINUTES = 60
SSH_ATTEMPTS = 5


def make_override_action(override_args):
    """Argparse action that remembers which options were given explicitly."""
    class StoreOverrideAction(argparse.Action):
        def __call__(self, parser, args, values, option_string=None):
            override_args.add(self.dest)
            setattr(args, self.dest, values)
    return StoreOverrideAction


def make_override_bool_action(override_args, bool_value):
    class StoreOverrideBoolAction(argparse.Action):
        def __init__(self, option_strings, dest, required=False, help=None, **kw):
            super().__init__(option_strings=option_strings, dest=dest, const=bool_value,
                             nargs=0, default=None, required=required, help=help)

        def __call__(self, parser, args, values, option_string=None):
            override_args.add(self.dest)
            setattr(args, self.dest, self.const)
    return StoreOverrideBoolAction


def make_override_true_action(override_args):
    return make_override_bool_action(override_args, True)


def make_override_false_action(override_args):
    return make_override_bool_action(override_args, False)


def check_build(verbose):
    """Prints what this build supports (``horovodrun --check-build``)."""
    def mark(v):
        return "[X]" if v else "[ ]"
    try:
        from horovod_b200 import _C  # noqa: F401
        native = True
    except ImportError:
        native = False
    try:
        import torch
        has_torch, cuda = True, torch.cuda.is_available()
    except ImportError:
        has_torch, cuda = False, False
    out = textwrap.dedent("""\
        horovod_b200 v{version}:

        Available Frameworks:
            {torch} PyTorch
            [ ] TensorFlow
            [ ] MXNet

        Available Controllers:
            [ ] MPI
            {native} TCP mesh + HTTP rendezvous (gloo-style)

        Available Tensor Operations:
            {native} NVLink symmetric-memory kernels (sm_100a)
            {native} NCCL (baseline / fallback)
            [ ] DDL
            [ ] CCL
            [ ] MPI
            {native} TCP mesh (CPU tensors)

        CUDA device visible: {cuda}""").format(
        version=horovod_b200.__version__, torch=mark(has_torch), native=mark(native),
        cuda="yes" if cuda else "no")
    print(out)
    sys.exit(0)


def parse_args(argv=None):
    override_args = set()
    parser = argparse.ArgumentParser(description="horovod_b200 launcher")
    parser.add_argument("-v", "--version", action="version", version=horovod_b200.__version__)
    np_arg = parser.add_argument("-np", "--num-proc", dest="np", type=int,
                                 action=make_override_action(override_args),
                                 help="Total number of training processes.")
    parser.add_argument("-cb", "--check-build", action="store_true", dest="check_build")
    parser.add_argument("--disable-cache", action="store_true", dest="disable_cache")
    parser.add_argument("--start-timeout", type=int, dest="start_timeout",
                        action=make_override_action(override_args))
    parser.add_argument("--network-interface", dest="nics",
                        action=make_override_action(override_args))
    parser.add_argument("--output-filename", dest="output_filename",
                        action=make_override_action(override_args))
    parser.add_argument("--verbose", action="store_true", dest="verbose")
    parser.add_argument("--config-file", dest="config_file",
                        action=make_override_action(override_args))
    parser.add_argument("-p", "--ssh-port", type=int, dest="ssh_port")
    parser.add_argument("-i", "--ssh-identity-file", dest="ssh_identity_file")
    parser.add_argument("command", nargs=argparse.REMAINDER)

    g = parser.add_argument_group("tunable parameter arguments")
    g.add_argument("--fusion-threshold-mb", type=int, dest="fusion_threshold_mb",
                   action=make_override_action(override_args))
    g.add_argument("--cycle-time-ms", type=float, dest="cycle_time_ms",
                   action=make_override_action(override_args))
    g.add_argument("--cache-capacity", type=int, dest="cache_capacity",
                   action=make_override_action(override_args))
    g.add_argument("--hierarchical-allreduce", dest="hierarchical_allreduce",
                   action=make_override_true_action(override_args))
    g.add_argument("--no-hierarchical-allreduce", dest="hierarchical_allreduce",
                   action=make_override_false_action(override_args))
    g.add_argument("--hierarchical-allgather", dest="hierarchical_allgather",
                   action=make_override_true_action(override_args))
    g.add_argument("--no-hierarchical-allgather", dest="hierarchical_allgather",
                   action=make_override_false_action(override_args))

    g = parser.add_argument_group("autotune arguments")
    g.add_argument("--autotune", dest="autotune", action=make_override_true_action(override_args))
    g.add_argument("--no-autotune", dest="autotune",
                   action=make_override_false_action(override_args))
    g.add_argument("--autotune-log-file", dest="autotune_log_file",
                   action=make_override_action(override_args))
    g.add_argument("--autotune-warmup-samples", type=int, dest="autotune_warmup_samples",
                   action=make_override_action(override_args))
    g.add_argument("--autotune-steps-per-sample", type=int, dest="autotune_steps_per_sample",
                   action=make_override_action(override_args))
    g.add_argument("--autotune-bayes-opt-max-samples", type=int,
                   dest="autotune_bayes_opt_max_samples",
                   action=make_override_action(override_args))
    g.add_argument("--autotune-gaussian-process-noise", type=float,
                   dest="autotune_gaussian_process_noise",
                   action=make_override_action(override_args))

    g = parser.add_argument_group("elastic arguments")
    g.add_argument("--min-np", "--min-num-proc", type=int, dest="min_np",
                   action=make_override_action(override_args))
    g.add_argument("--max-np", "--max-num-proc", type=int, dest="max_np",
                   action=make_override_action(override_args))
    g.add_argument("--slots-per-host", "--slots", type=int, dest="slots",
                   action=make_override_action(override_args))
    g.add_argument("--elastic-timeout", type=int, dest="elastic_timeout",
                   action=make_override_action(override_args))
    g.add_argument("--reset-limit", type=int, dest="reset_limit",
                   action=make_override_action(override_args))

    g = parser.add_argument_group("timeline arguments")
    g.add_argument("--timeline-filename", dest="timeline_filename",
                   action=make_override_action(override_args))
    g.add_argument("--timeline-mark-cycles", dest="timeline_mark_cycles",
                   action=make_override_true_action(override_args))
    g.add_argument("--no-timeline-mark-cycles", dest="timeline_mark_cycles",
                   action=make_override_false_action(override_args))

    g = parser.add_argument_group("stall check arguments")
    g.add_argument("--no-stall-check", dest="no_stall_check",
                   action=make_override_true_action(override_args))
    g.add_argument("--stall-check", dest="no_stall_check",
                   action=make_override_false_action(override_args))
    g.add_argument("--stall-check-warning-time-seconds", type=int,
                   dest="stall_check_warning_time_seconds",
                   action=make_override_action(override_args))
    g.add_argument("--stall-check-shutdown-time-seconds", type=int,
                   dest="stall_check_shutdown_time_seconds",
                   action=make_override_action(override_args))

    g = parser.add_argument_group("library arguments")
    g.add_argument("--num-nccl-streams", type=int, dest="num_nccl_streams",
                   action=make_override_action(override_args))
    g.add_argument("--gloo-timeout-seconds", type=int, dest="gloo_timeout_seconds",
                   action=make_override_action(override_args),
                   help="Timeout of the control-plane (TCP mesh) operations, default 30.")
    g.add_argument("--thread-affinity", type=int, dest="thread_affinity",
                   action=make_override_action(override_args))
    g.add_argument("--gpu-backend", dest="gpu_backend", choices=["symm", "nccl"],
                   action=make_override_action(override_args),
                   help="Device data path: NVLink kernels (default) or NCCL.")

    g = parser.add_argument_group("logging arguments")
    g.add_argument("--log-level", dest="log_level", choices=config_parser.LOG_LEVELS,
                   action=make_override_action(override_args))
    # Timestamps inside the library's own log lines: the positive and the
    # negative spelling, plus the older "hide" pair with the opposite sense.
    g.add_argument("--log-with-timestamp", dest="log_hide_timestamp",
                   action=make_override_false_action(override_args),
                   help="Keep the timestamp in the library's log messages (the default).")
    g.add_argument("--log-without-timestamp", dest="log_hide_timestamp",
                   action=make_override_true_action(override_args),
                   help="Hide the timestamp from the library's log messages.")
    g.add_argument("--log-hide-timestamp", dest="log_hide_timestamp",
                   action=make_override_true_action(override_args), help=argparse.SUPPRESS)
    g.add_argument("--no-log-hide-timestamp", dest="log_hide_timestamp",
                   action=make_override_false_action(override_args), help=argparse.SUPPRESS)
    g.add_argument("-prefix-timestamp", "--prefix-output-with-timestamp", "--prefix-timestamp",
                   dest="prefix_output_with_timestamp", action="store_true",
                   help="Timestamp each line of the workers' output.")

    g = parser.add_argument_group("host arguments")
    hx = g.add_mutually_exclusive_group()
    hx.add_argument("-H", "--hosts", dest="hosts", action=make_override_action(override_args),
                    help="host1:slots,host2:slots")
    hx.add_argument("-hostfile", "--hostfile", dest="hostfile",
                    action=make_override_action(override_args))
    hx.add_argument("--host-discovery-script", dest="host_discovery_script",
                    action=make_override_action(override_args))

    g = parser.add_argument_group("controller arguments")
    cx = g.add_mutually_exclusive_group()
    cx.add_argument("--gloo", action="store_true", dest="use_gloo")
    cx.add_argument("--mpi", action="store_true", dest="use_mpi")
    cx.add_argument("--jsrun", action="store_true", dest="use_jsrun")
    tx = g.add_mutually_exclusive_group()
    tx.add_argument("--mpi-threads-disable", dest="mpi_threads_disable",
                    action=make_override_true_action(override_args),
                    help="Passed on as HOROVOD_MPI_THREADS_DISABLE; only meaningful for jobs "
                         "started through mpirun, this runtime has no MPI threads of its own.")
    tx.add_argument("--no-mpi-threads-disable", dest="mpi_threads_disable",
                    action=make_override_false_action(override_args), help=argparse.SUPPRESS)
    g.add_argument("--mpi-args", dest="mpi_args")
    g.add_argument("--tcp", action="store_true", dest="tcp_flag")
    g.add_argument("--binding-args", dest="binding_args")

    args = parser.parse_args(argv)
    if args.config_file:
        with open(args.config_file) as f:
            config = yaml.safe_load(f) or {}
        config_parser.set_args_from_config(args, config, override_args)
    config_parser.validate_config_args(args)
    args.run_func = None
    if not args.check_build and not args.command and not getattr(args, "run_func", None):
        parser.error("the following arguments are required: command")
    if not args.check_build and args.np is None and args.min_np is None:
        raise argparse.ArgumentError(np_arg, "-np (or --min-np for elastic jobs) is required")
    return args


def _ssh_reachable(host, port, identity, timeout_s):
    import subprocess
    opts = ["-o", "PasswordAuthentication=no", "-o", "StrictHostKeyChecking=no",
            "-o", "ConnectTimeout=%d" % timeout_s]
    if port:
        opts += ["-p", str(port)]
    if identity:
        opts += ["-i", identity]
    for _ in range(SSH_ATTEMPTS):
        try:
            if subprocess.call(["ssh"] + opts + [host, "true"], stdout=subprocess.DEVNULL,
                               stderr=subprocess.DEVNULL, timeout=timeout_s + 5) == 0:
                return True
        except (OSError, subprocess.TimeoutExpired):
            pass
    return False


def check_all_hosts_ssh_successful(host_names, ssh_port=None, ssh_identity_file=None,
                                   fn_cache=None):
    """Every remote host must accept password-less ssh; results are cached."""
    bad = []
    for h in host_names:
        key = ("ssh", h, ssh_port, ssh_identity_file)
        ok = fn_cache.get(key) if fn_cache else None
        if ok is None:
            ok = _ssh_reachable(h, ssh_port, ssh_identity_file, 10)
            if fn_cache:
                fn_cache.put(key, ok)
        if not ok:
            bad.append(h)
    if bad:
        raise RuntimeError("could not connect to some hosts via ssh: %s" % ", ".join(bad))
    return True


def _build_settings(args):
    if args.hostfile:
        args.hosts = hosts_mod.parse_host_files(args.hostfile)
    elastic = bool(args.host_discovery_script) or args.min_np is not None or \
        args.max_np is not None
    tmout = Timeout(args.start_timeout or int(os.environ.get("HOROVOD_START_TIMEOUT", "30")),
                    message="Timed out waiting for {activity}. Please check connectivity "
                            "between servers. You may need to increase the --start-timeout "
                            "parameter if you have too many servers.")
    common = dict(num_proc=args.np, verbose=2 if args.verbose else 0, ssh_port=args.ssh_port,
                  ssh_identity_file=args.ssh_identity_file, extra_mpi_args=args.mpi_args,
                  tcp_flag=args.tcp_flag, binding_args=args.binding_args,
                  start_timeout=tmout, output_filename=args.output_filename,
                  run_func_mode=args.run_func is not None, nics=args.nics,
                  prefix_output_with_timestamp=args.prefix_output_with_timestamp)
    if elastic:
        from horovod_b200.runner.elastic import discovery
        if args.host_discovery_script:
            disc = discovery.HostDiscoveryScript(args.host_discovery_script, args.slots)
        elif args.hosts:
            disc = discovery.FixedHosts({h.hostname: h.slots
                                         for h in hosts_mod.parse_hosts(args.hosts)})
        else:
            disc = discovery.FixedHosts({"localhost": args.max_np or args.np or args.min_np})
        min_np = args.min_np or args.np
        common["num_proc"] = args.np or min_np
        return ElasticSettings(discovery=disc, min_np=min_np, max_np=args.max_np,
                               elastic_timeout=args.elastic_timeout or 600,
                               reset_limit=args.reset_limit, **common)
    if not args.hosts:
        args.hosts = "localhost:%d" % args.np
    return Settings(hosts=args.hosts, **common)


def _run(args):
    if args.check_build:
        check_build(args.verbose)
    settings = _build_settings(args)
    env = os.environ.copy()
    config_parser.set_env_from_args(env, args)
    # Workers must import this very package.
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")

    if args.use_mpi or args.use_jsrun:
        from horovod_b200.runner import mpi_run, js_run
        if args.use_mpi:
            return mpi_run.mpi_run(settings, args.nics, env, args.command)
        return js_run.js_run(settings, args.nics, env, args.command)

    if settings.elastic:
        return gloo.gloo_run_elastic(settings, env, args.command)

    host_names = [h.hostname for h in hosts_mod.parse_hosts(settings.hosts)]
    remote = [h for h in host_names if not gloo.is_local_host(h)]
    if remote:
        fn_cache = None if args.disable_cache else cache_mod.Cache(
            CACHE_FOLDER, CACHE_STALENESS_THRESHOLD_MINUTES, (settings.hosts,))
        check_all_hosts_ssh_successful(remote, args.ssh_port, args.ssh_identity_file, fn_cache)
        from horovod_b200.runner.http.http_server import local_ip_for
        server_ip = local_ip_for(remote[0])
    else:
        server_ip = "127.0.0.1"
    nics = set(args.nics.split(",")) if args.nics else None
    if remote and nics is None:
        # Find the interfaces that are routed between all hosts (each host's
        # task service probes the next one's); cached per host list.
        from horovod_b200.runner.driver import driver_service
        local = [h for h in host_names if gloo.is_local_host(h)]

        def discover():
            return sorted(driver_service.get_common_interfaces(
                host_names, local_host_names=local, ssh_port=args.ssh_port,
                ssh_identity_file=args.ssh_identity_file,
                start_timeout_s=max(1, int(settings.start_timeout.remaining()))
                if settings.start_timeout is not None else 30))
        try:
            if fn_cache is not None:
                found = fn_cache.get(("nics",) + tuple(host_names))
                if found is None:
                    found = discover()
                    fn_cache.put(("nics",) + tuple(host_names), found)
            else:
                found = discover()
            nics = set(found)
        except Exception as e:  # noqa: BLE001 - discovery is best effort
            if settings.verbose:
                print("NIC discovery failed (%s); letting the ranks pick their interface." % e)
    return gloo.gloo_run(settings, nics, env, server_ip, args.command)


def run_commandline(argv=None):
    args = parse_args(argv)
    try:
        _run(args)
    except RuntimeError as e:
        print(str(e), file=sys.stderr)
        sys.exit(1)


if __name__ == "__main__":
    run_commandline()
