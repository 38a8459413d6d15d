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
    # ---- the fused form: the attention launch itself stores into the peers' rows ----------------
    qh, kvh, hd = 8, 2, 128                      # this rank's heads
    kv_dim, q_dim = kvh * hd, qh * hd
    assert n * q_dim <= row
    for ctx in (40, 700, 9000):                  # one split; cluster-sized; shared merge
        n_steps = 60 if ctx == 9000 else 24    # many exchanges: a store that overtook its flag would show as a stale slice
        cap = ctx + n_steps + 16
        pool = st.pool(1, kvh, hd, sg.KV_BF16, num_pages=2 * (cap // 16 + 2), max_seqs=2, max_seq_tokens=cap)
        seqs = [pool.sequence(cap) for _ in range(2)]          # twin sequences: one decodes through the exchange
        kvs = [sq.layer(0, qh) for sq in seqs]
        d_k, d_v = st.alloc(4 * ctx * kv_dim), st.alloc(4 * ctx * kv_dim)
        st.fill_normal(d_k, ctx * kv_dim, 60 + rank, 0)
        st.fill_normal(d_v, ctx * kv_dim, 60 + rank, 1)
        for kv in kvs:
            kv.encode_append_rows(d_k, d_v, ctx)
        st.sync()
        b_ex, b_plain = sg.Batch(st, [kvs[0]]), sg.Batch(st, [kvs[1]])
        d_kn, d_vn, d_q, d_o = st.alloc(4 * kv_dim), st.alloc(4 * kv_dim), st.alloc(4 * q_dim), st.alloc(4 * q_dim)
        for step in range(n_steps):
            st.fill_normal(d_kn, kv_dim, 70 + rank, 3 * step)
            st.fill_normal(d_vn, kv_dim, 70 + rank, 3 * step + 1)
            st.fill_normal(d_q, q_dim, 70 + rank, 3 * step + 2)
            off = (step % 2) * layers * row          # row 0 of either set
            peer_rows = [0 if p == rank else peers[p].ptr + 4 * off for p in range(n)]
            b_ex.enqueue_step_exchange(d_kn, d_vn, d_q, ex, rows.ptr + 4 * off, peer_rows, rank * q_dim)
            b_plain.enqueue_step(d_kn, d_vn, d_q, d_o)
            st.sync()
            assert st.device_status() == 0
            own = d_o.download(np.float32, q_dim)
            put(os.path.join(d, f"slice_{ctx}_{step}_{rank}"), own.tobytes())
            got = rows.download(np.float32, 2 * layers * row)[off:off + n * q_dim].reshape(n, q_dim)
            for p in range(n):
                want = np.frombuffer(get(os.path.join(d, f"slice_{ctx}_{step}_{p}"), deadline), np.float32)
                assert np.array_equal(got[p], want), (ctx, step, p)
        b_ex.close()
        b_plain.close()
        for sq in seqs:
            sq.close()
        pool.close()
    # ---- a peer that stops joining: the last rank skips one exchange (it stays alive, its rows and
    # flags stay mapped); the others' wait for its flag runs out on the device after a second or
    # so, the kernel reports through the status word and returns, and the context stays usable.
    # Nothing faults and nothing hangs: the failure is made on the host.
    if rank != n - 1:
        off = 0
        peer_rows = [0 if p == rank else peers[p].ptr + 4 * off for p in range(n)]
        t0 = time.time()
        ex.enqueue(rows.ptr + 4 * off, peer_rows, rank * sl, sl)
        st.sync()
        waited = time.time() - t0
        status = st.device_status()                      # reads and clears
        assert status == 6, status                      # SGK_ERR_TIMEOUT: a bounded device-side wait expired
        assert waited < 30.0, waited
        assert st.device_status() == 0
        probe = st.alloc(4 * 64)
        probe.upload(np.arange(64, dtype=np.float32))
        assert np.array_equal(probe.download(np.float32, 64), np.arange(64, dtype=np.float32))
        print(f"TIMEOUT-REPORTED after {waited:.2f} s", flush=True)
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
