"""Stand-in: cluster detection is not used by the benchmark arm."""


def get_job():
    raise RuntimeError("clusterscope is not available")


def cluster():
    return "local"
