"""Runs fused append + attention steps at forced split counts and saves the outputs; the parent test
runs it twice, with and without SGK_NO_CLUSTER_MERGE, and compares the files bit for bit."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import saragossa_b200 as sg  # noqa: E402


def main(out_path):
    st = sg.DecodeResidentState(0)
    outs = {}
    cases = [(32, 8, 128, sg.KV_BF16, 700), (16, 2, 256, sg.KV_BF16, 530), (32, 4, 128, sg.KV_BF16, 1500),
             (16, 2, 256, sg.KV_U8G32, 700), (8, 8, 128, sg.KV_BF16, 333)]
    for ci, (qh, kvh, hd, dtype, ctx) in enumerate(cases):
        kv_dim, q_dim = kvh * hd, qh * hd
        for n_seq in (1, 3):
            cap = ctx + 64
            pool = st.pool(1, kvh, hd, dtype, num_pages=n_seq * (cap // 16 + 2), max_seqs=n_seq, max_seq_tokens=cap)
            pool.shuffle_free_list(ci)
            seqs = [pool.sequence(cap) for _ in range(n_seq)]
            kvs = [seq.layer(0, qh) for seq in seqs]
            for s, kv in enumerate(kvs):
                rows = ctx - 37 * s   # ragged batch
                d_k, d_v = st.alloc(4 * rows * kv_dim), st.alloc(4 * rows * kv_dim)
                st.fill_normal(d_k, rows * kv_dim, 40 + ci, 2 * s)
                st.fill_normal(d_v, rows * kv_dim, 40 + ci, 2 * s + 1)
                kv.encode_append_rows(d_k, d_v, rows)
            st.sync()
            batch = sg.Batch(st, kvs)
            d_kn, d_vn = st.alloc(4 * n_seq * kv_dim), st.alloc(4 * n_seq * kv_dim)
            d_q, d_o = st.alloc(4 * n_seq * q_dim), st.alloc(4 * n_seq * q_dim)
            for splits in (2, 3, 5, 8, 11, 16):
                batch.set_splits(splits)
                for step in range(2):
                    st.fill_normal(d_kn, n_seq * kv_dim, 50 + ci, 3 * step)
                    st.fill_normal(d_vn, n_seq * kv_dim, 50 + ci, 3 * step + 1)
                    st.fill_normal(d_q, n_seq * q_dim, 50 + ci, 3 * step + 2)
                    batch.enqueue_step(d_kn, d_vn, d_q, d_o)
                    st.sync()
                    assert batch.last_splits() == splits
                    outs[f"c{ci}_n{n_seq}_s{splits}_t{step}"] = d_o.download(count=n_seq * q_dim).copy()
            batch.close()
            for seq in seqs:
                seq.close()
            pool.close()
    assert st.device_status() == 0
    np.savez(out_path, **outs)
    st.close()


if __name__ == "__main__":
    main(sys.argv[1])
