"""Maps launcher options (CLI flags or a YAML config file) onto the
HOROVOD_* environment variables the runtime reads at init. Precedence is
explicit flag > config file > default.

Parity: horovod/runner/common/util/config_parser.py:55-202.
"""
# Environment variable names (shared with csrc/common/env.h).
HOROVOD_FUSION_THRESHOLD = "HOROVOD_FUSION_THRESHOLD"
HOROVOD_CYCLE_TIME = "HOROVOD_CYCLE_TIME"
HOROVOD_CACHE_CAPACITY = "HOROVOD_CACHE_CAPACITY"
HOROVOD_HIERARCHICAL_ALLREDUCE = "HOROVOD_HIERARCHICAL_ALLREDUCE"
HOROVOD_HIERARCHICAL_ALLGATHER = "HOROVOD_HIERARCHICAL_ALLGATHER"
HOROVOD_AUTOTUNE = "HOROVOD_AUTOTUNE"
HOROVOD_AUTOTUNE_LOG = "HOROVOD_AUTOTUNE_LOG"
HOROVOD_AUTOTUNE_WARMUP_SAMPLES = "HOROVOD_AUTOTUNE_WARMUP_SAMPLES"
HOROVOD_AUTOTUNE_STEPS_PER_SAMPLE = "HOROVOD_AUTOTUNE_STEPS_PER_SAMPLE"
HOROVOD_AUTOTUNE_BAYES_OPT_MAX_SAMPLES = "HOROVOD_AUTOTUNE_BAYES_OPT_MAX_SAMPLES"
HOROVOD_AUTOTUNE_GAUSSIAN_PROCESS_NOISE = "HOROVOD_AUTOTUNE_GAUSSIAN_PROCESS_NOISE"
HOROVOD_TIMELINE = "HOROVOD_TIMELINE"
HOROVOD_TIMELINE_MARK_CYCLES = "HOROVOD_TIMELINE_MARK_CYCLES"
HOROVOD_STALL_CHECK_DISABLE = "HOROVOD_STALL_CHECK_DISABLE"
HOROVOD_STALL_CHECK_TIME_SECONDS = "HOROVOD_STALL_CHECK_TIME_SECONDS"
HOROVOD_STALL_SHUTDOWN_TIME_SECONDS = "HOROVOD_STALL_SHUTDOWN_TIME_SECONDS"
HOROVOD_LOG_LEVEL = "HOROVOD_LOG_LEVEL"
HOROVOD_LOG_HIDE_TIME = "HOROVOD_LOG_HIDE_TIME"
HOROVOD_GLOO_TIMEOUT_SECONDS = "HOROVOD_GLOO_TIMEOUT_SECONDS"
HOROVOD_MPI_THREADS_DISABLE = "HOROVOD_MPI_THREADS_DISABLE"
HOROVOD_NUM_NCCL_STREAMS = "HOROVOD_NUM_NCCL_STREAMS"
HOROVOD_THREAD_AFFINITY = "HOROVOD_THREAD_AFFINITY"
HOROVOD_GPU_BACKEND = "HOROVOD_GPU_BACKEND"

LOG_LEVELS = ["TRACE", "DEBUG", "INFO", "WARNING", "ERROR", "FATAL"]


def _set_arg_from_config(args, arg_base_name, override_args, config, arg_prefix=""):
    arg_name = arg_prefix + arg_base_name
    if arg_name in override_args:
        return  # the command line wins
    value = config.get(arg_base_name)
    if value is not None:
        setattr(args, arg_name, value)


def set_args_from_config(args, config, override_args):
    """Copies values of the parsed YAML ``config`` into ``args`` unless the
    flag was given on the command line (``override_args``)."""
    params = config.get("params")
    if params:
        for k in ("fusion_threshold_mb", "cycle_time_ms", "cache_capacity",
                  "hierarchical_allreduce", "hierarchical_allgather"):
            _set_arg_from_config(args, k, override_args, params)
    library_options = config.get("library_options")
    if library_options:
        _set_arg_from_config(args, "mpi_threads_disable", override_args, library_options)
    autotune = config.get("autotune")
    if autotune:
        args.autotune = autotune.get("enabled", False) \
            if "autotune" not in override_args else args.autotune
        for k in ("log_file", "warmup_samples", "steps_per_sample", "bayes_opt_max_samples",
                  "gaussian_process_noise"):
            _set_arg_from_config(args, k, override_args, autotune, arg_prefix="autotune_")
    timeline = config.get("timeline")
    if timeline:
        _set_arg_from_config(args, "filename", override_args, timeline, arg_prefix="timeline_")
        _set_arg_from_config(args, "mark_cycles", override_args, timeline,
                             arg_prefix="timeline_")
    stall = config.get("stall_check")
    if stall:
        args.no_stall_check = not stall.get("enabled", True) \
            if "no_stall_check" not in override_args else args.no_stall_check
        _set_arg_from_config(args, "warning_time_seconds", override_args, stall,
                             arg_prefix="stall_check_")
        _set_arg_from_config(args, "shutdown_time_seconds", override_args, stall,
                             arg_prefix="stall_check_")
    library = config.get("library_options")
    if library:
        _set_arg_from_config(args, "num_nccl_streams", override_args, library)
        _set_arg_from_config(args, "thread_affinity", override_args, library)
        _set_arg_from_config(args, "gloo_timeout_seconds", override_args, library)
        _set_arg_from_config(args, "gpu_backend", override_args, library)
    logging = config.get("logging")
    if logging:
        _set_arg_from_config(args, "level", override_args, logging, arg_prefix="log_")
        _set_arg_from_config(args, "hide_timestamp", override_args, logging, arg_prefix="log_")
        if "with_timestamp" in logging and "log_hide_timestamp" not in override_args:
            args.log_hide_timestamp = not logging["with_timestamp"]


def validate_config_args(args):
    def need(cond, msg):
        if not cond:
            raise ValueError(msg)
    if getattr(args, "fusion_threshold_mb", None) is not None:
        need(args.fusion_threshold_mb >= 0, "fusion_threshold_mb must be >= 0")
    if getattr(args, "cycle_time_ms", None) is not None:
        need(args.cycle_time_ms > 0, "cycle_time_ms must be > 0")
    if getattr(args, "cache_capacity", None) is not None:
        need(args.cache_capacity >= 0, "cache_capacity must be >= 0")
    for name in ("autotune_warmup_samples", "autotune_steps_per_sample",
                 "autotune_bayes_opt_max_samples"):
        v = getattr(args, name, None)
        if v is not None:
            need(v > 0 if name != "autotune_warmup_samples" else v >= 0,
                 "%s must be positive" % name)
    v = getattr(args, "autotune_gaussian_process_noise", None)
    if v is not None:
        need(0 <= v <= 1, "autotune_gaussian_process_noise must be in [0, 1]")
    w = getattr(args, "stall_check_warning_time_seconds", None)
    s = getattr(args, "stall_check_shutdown_time_seconds", None)
    t = getattr(args, "gloo_timeout_seconds", None)
    if t is not None:
        need(t >= 0, "gloo_timeout_seconds must be >= 0")
    if w is not None:
        need(w >= 0, "stall_check_warning_time_seconds must be >= 0")
    if s is not None:
        need(s >= 0, "stall_check_shutdown_time_seconds must be >= 0")


def _add(env, name, value, transform=str):
    if value is not None and value is not False:
        env[name] = transform(value)


def set_env_from_args(env, args):
    """Writes the HOROVOD_* variables for every option that is set."""
    def g(name):
        return getattr(args, name, None)
    _add(env, HOROVOD_FUSION_THRESHOLD, g("fusion_threshold_mb"),
         lambda v: str(int(v * 1024 * 1024)))
    _add(env, HOROVOD_CYCLE_TIME, g("cycle_time_ms"))
    _add(env, HOROVOD_CACHE_CAPACITY, g("cache_capacity"))
    _add(env, HOROVOD_HIERARCHICAL_ALLREDUCE, g("hierarchical_allreduce"), lambda v: "1")
    _add(env, HOROVOD_HIERARCHICAL_ALLGATHER, g("hierarchical_allgather"), lambda v: "1")
    if g("autotune"):
        env[HOROVOD_AUTOTUNE] = "1"
        _add(env, HOROVOD_AUTOTUNE_LOG, g("autotune_log_file"))
        _add(env, HOROVOD_AUTOTUNE_WARMUP_SAMPLES, g("autotune_warmup_samples"))
        _add(env, HOROVOD_AUTOTUNE_STEPS_PER_SAMPLE, g("autotune_steps_per_sample"))
        _add(env, HOROVOD_AUTOTUNE_BAYES_OPT_MAX_SAMPLES, g("autotune_bayes_opt_max_samples"))
        _add(env, HOROVOD_AUTOTUNE_GAUSSIAN_PROCESS_NOISE,
             g("autotune_gaussian_process_noise"))
    _add(env, HOROVOD_TIMELINE, g("timeline_filename"))
    _add(env, HOROVOD_TIMELINE_MARK_CYCLES, g("timeline_mark_cycles"), lambda v: "1")
    _add(env, HOROVOD_STALL_CHECK_DISABLE, g("no_stall_check"), lambda v: "1")
    _add(env, HOROVOD_STALL_CHECK_TIME_SECONDS, g("stall_check_warning_time_seconds"))
    _add(env, HOROVOD_STALL_SHUTDOWN_TIME_SECONDS, g("stall_check_shutdown_time_seconds"))
    _add(env, HOROVOD_MPI_THREADS_DISABLE, g("mpi_threads_disable"), lambda v: "1")
    _add(env, HOROVOD_NUM_NCCL_STREAMS, g("num_nccl_streams"))
    _add(env, HOROVOD_THREAD_AFFINITY, g("thread_affinity"))
    _add(env, HOROVOD_GLOO_TIMEOUT_SECONDS, g("gloo_timeout_seconds"))
    _add(env, HOROVOD_GPU_BACKEND, g("gpu_backend"))
    _add(env, HOROVOD_LOG_LEVEL, g("log_level"))
    _add(env, HOROVOD_LOG_HIDE_TIME, g("log_hide_timestamp"), lambda v: "1")
    return env
