"""Worker: the link probe on CPU ranks."""
import json
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from dew_b200.parallel.probe import communicator_memory, probe  # noqa: E402


def main():
    dist.init_process_group("gloo")
    link = probe(sizes=(1 << 16, 1 << 18), iters=2)
    mem = communicator_memory()
    if dist.get_rank() == 0:
        print("RESULT " + json.dumps({"rows": len(link.rows), "names": sorted({r.collective for r in link.rows}),
                                      "positive": all(r.ms > 0 and r.busbw_gbs > 0 for r in link.rows), "mem": mem["bytes"],
                                      "table_lines": len(link.table().splitlines()), "spread": link.spread_pays(1e9)}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
