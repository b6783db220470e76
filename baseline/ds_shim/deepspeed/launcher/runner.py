"""Host-file helpers the reference imports at module scope (single-node stand-in)."""
import collections
import os

DLTS_HOSTFILE = "/job/hostfile"


def fetch_hostfile(path):
    if not path or not os.path.isfile(path):
        return None
    pool = collections.OrderedDict()
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            host, slots = line.split()
            pool[host] = int(slots.split("=")[1])
    return pool


def parse_inclusion_exclusion(resource_pool, inclusion, exclusion):
    return collections.OrderedDict((h, list(range(n))) for h, n in (resource_pool or {}).items())
