def mpi_discovery(*a, **k):
    raise RuntimeError("MPI discovery is not provided by the deepspeed stand-in")
