"""Entry point of ranks started by mpirun/jsrun: translates the MPI
launcher's rank variables into the HOROVOD_* ones and execs the command."""
import os
import sys


def main():
    addr, port, command = sys.argv[1], sys.argv[2], sys.argv[3:]
    env = os.environ

    def first(*names, default="0"):
        for n in names:
            if n in env:
                return env[n]
        return default
    rank = first("OMPI_COMM_WORLD_RANK", "PMI_RANK", "PMIX_RANK", "JSM_NAMESPACE_RANK")
    size = first("OMPI_COMM_WORLD_SIZE", "PMI_SIZE", "JSM_NAMESPACE_SIZE", default="1")
    lrank = first("OMPI_COMM_WORLD_LOCAL_RANK", "MPI_LOCALRANKID", "JSM_NAMESPACE_LOCAL_RANK")
    lsize = first("OMPI_COMM_WORLD_LOCAL_SIZE", "MPI_LOCALNRANKS", "JSM_NAMESPACE_LOCAL_SIZE",
                  default="1")
    env.update({
        "HOROVOD_RANK": rank, "HOROVOD_SIZE": size, "HOROVOD_LOCAL_RANK": lrank,
        "HOROVOD_LOCAL_SIZE": lsize,
        "HOROVOD_CROSS_RANK": str(int(rank) // max(1, int(lsize))),
        "HOROVOD_CROSS_SIZE": str(max(1, int(size) // max(1, int(lsize)))),
        "HOROVOD_GLOO_RENDEZVOUS_ADDR": addr, "HOROVOD_GLOO_RENDEZVOUS_PORT": port,
    })
    os.execvp(command[0], command)


if __name__ == "__main__":
    main()
