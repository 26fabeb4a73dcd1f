"""LSF (jsrun) environment: hosts and slots of the current allocation.
Parity: horovod/runner/util/lsf.py:26-103."""
import os


class LSFUtils:
    """Reads the compute hosts of an LSF job from LSB_MCPU_HOSTS /
    LSB_DJOB_HOSTFILE (the first host is the launch node and is skipped when
    the allocation has batch nodes)."""

    @staticmethod
    def using_lsf():
        return "LSB_JOBID" in os.environ

    @staticmethod
    def get_compute_hosts():
        mcpu = os.environ.get("LSB_MCPU_HOSTS", "").split()
        hosts = []
        for name in mcpu[0::2]:
            if name not in hosts:
                hosts.append(name)
        if not hosts and os.environ.get("LSB_DJOB_HOSTFILE"):
            with open(os.environ["LSB_DJOB_HOSTFILE"]) as f:
                for line in f:
                    name = line.strip()
                    if name and name not in hosts:
                        hosts.append(name)
        # batch/launch node first
        return hosts[1:] if len(hosts) > 1 else hosts

    @staticmethod
    def get_num_gpus():
        """GPUs per host, from the visible devices of the launch environment."""
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            return len([d for d in visible.split(",") if d.strip()])
        try:
            import torch
            return torch.cuda.device_count()
        except Exception:  # noqa: BLE001
            return 0

    @staticmethod
    def get_num_cores():
        return os.cpu_count() or 1

    @staticmethod
    def get_num_threads():
        return 1

    @staticmethod
    def get_num_processes():
        return len(LSFUtils.get_compute_hosts()) * max(1, LSFUtils.get_num_gpus())
