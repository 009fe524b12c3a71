"""One process of the symmetric-allocator test (host stand-in: memfd-backed memory, real descriptor passing)."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.parallel.symm_alloc import SymmetricAllocation  # noqa: E402


def main():
    rank, world, job, sock_dir, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5]
    a = SymmetricAllocation(10_000, rank, world, job=job, sock_dir=sock_dir, host=True, timeout_s=30)
    assert a.bytes_per_rank >= 10_000 and a.bytes_per_rank % 4096 == 0
    assert all(a.ptrs[r + 1] - a.ptrs[r] == a.bytes_per_rank for r in range(world - 1))
    mine = a.tensor(dtype=torch.int32)
    mine[:16] = torch.arange(16, dtype=torch.int32) + 1000 * (rank + 1)       # my slot, through my mapping
    flags = a.tensor(dtype=torch.int32)
    flags[100] = 1                                                             # "my data is written"
    ok = True
    for peer in range(world):                                                  # every peer's slot, through MY mapping of it
        t = a.tensor(peer, dtype=torch.int32)
        t0 = time.time()
        while int(t[100]) != 1:
            if time.time() - t0 > 30:
                ok = False
                break
            time.sleep(0.01)
        ok = ok and bool(torch.equal(t[:16], torch.arange(16, dtype=torch.int32) + 1000 * (peer + 1)))
    # a store into a peer's slot is seen by the peer (what a kernel's peer store does)
    nxt = a.tensor((rank + 1) % world, dtype=torch.int32)
    nxt[200 + rank] = 77 + rank
    t0 = time.time()
    prev = (rank - 1) % world
    while int(mine[200 + prev]) != 77 + prev and time.time() - t0 < 30:
        time.sleep(0.01)
    ok = ok and int(mine[200 + prev]) == 77 + prev
    with open(out, "w") as f:
        f.write("ok" if ok else "bad")
    time.sleep(0.3)                    # let the peers finish reading before the mappings go away
    a.close()


if __name__ == "__main__":
    main()
