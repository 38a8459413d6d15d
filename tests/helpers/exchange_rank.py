"""One rank of the exchange test: python exchange_rank.py <rank> <n_ranks> <dir>. Handles travel through
files in <dir>; every wait on a file has a deadline. Prints OK on success."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import saragossa_b200 as sg  # noqa: E402


def put(path, data: bytes):
    with open(path + ".tmp", "wb") as f:
        f.write(data)
    os.replace(path + ".tmp", path)


def get(path, deadline):
    while not os.path.exists(path):
        if time.time() > deadline:
            raise TimeoutError(path)
        time.sleep(0.01)
    return open(path, "rb").read()


def main(rank, n, d):
    deadline = time.time() + 120
    st = sg.DecodeResidentState(rank)
    layers, row = 6, 4096                    # 2 x 6 rows of 4096 floats; a rank owns row/n of each
    sl = row // n
    rows = st.alloc(4 * 2 * layers * row)    # two sets of rows: a peer may be one exchange ahead
    rows.upload(np.zeros(2 * layers * row, np.float32))
    ex = st.exchange(rank, n)
    put(os.path.join(d, f"rows{rank}"), st.peer_export(rows))
    put(os.path.join(d, f"flags{rank}"), ex.handle)
    peers = {}
    for p in range(n):
        if p == rank:
            continue
        peers[p] = st.peer_open(get(os.path.join(d, f"rows{p}"), deadline))
        ex.connect(p, get(os.path.join(d, f"flags{p}"), deadline))
    steps = 7
    for step in range(steps):
        base = (step % 2) * layers * row
        for layer in range(layers):
            val = (np.arange(sl, dtype=np.float32) + 1000.0 * rank + 10.0 * layer + 100000.0 * step)
            off = base + layer * row
            # the rank's own slice lands in its row the way the attention kernel's output would
            sg.resident.check(st.L.sgk_util_h2d(st.h, rows.ptr + 4 * (off + rank * sl), val.ctypes.data, 4 * sl))
            peer_rows = [0 if p == rank else peers[p].ptr + 4 * off for p in range(n)]
            ex.enqueue(rows.ptr + 4 * off, peer_rows, rank * sl, sl)
        st.sync()
        assert st.device_status() == 0
        got = rows.download(np.float32, 2 * layers * row)[base:base + layers * row].reshape(layers, n, sl)
        for layer in range(layers):
            for p in range(n):
                want = np.arange(sl, dtype=np.float32) + 1000.0 * p + 10.0 * layer + 100000.0 * step
                assert np.array_equal(got[layer, p], want), (step, layer, p)
    # everybody done before anybody unmaps
    put(os.path.join(d, f"done{rank}"), b"1")
    for p in range(n):
        get(os.path.join(d, f"done{p}"), deadline)
    for p in peers.values():
        st.peer_close(p)
    ex.close()
    st.close()
    print("OK", flush=True)


if __name__ == "__main__":
    main(int(sys.argv[1]), int(sys.argv[2]), sys.argv[3])
