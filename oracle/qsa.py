"""CPU restatement (numpy, float64) of the reference's query-sparse paged attention.  TEST
INFRASTRUCTURE: only tests and the fixture generator import it; the product never does.

Follows crates/warp34-kernels/csrc/ops/op_qsa.cu:716-1075 (GQA kernel), :1076-1155 (split merge) and
:1450-1572 (launcher): every token attends to its list of selected 4-token groups,

    physical group id  -> page = id // 4, rows 4 (id % 4) .. + 3 of that page         (negative id: skipped)
    logical group      -> key position 4 * logical + off, visible iff <= token_seq_pos[token]

then softmax over the visible keys, output = P V, for rotated layers the inverse Walsh-Hadamard and the
sign diagonal, an optional sigmoid gate on the un-rounded result, and in the Hadamard variant a
normalised 64-point Hadamard over every 64 columns of the fp16-rounded gated values.  A token that
valid_token_mask switches off gets zero rows.

Pinned by tests/golden/qsa_ref_sm100a.npz: outputs of the reference's own kernels (compiled unmodified
into oracle/_ref) on a B200, produced by tests/golden/make_golden_qsa.py.
"""
import numpy as np

TQ4, Q8_0, FP8_E4M3 = 2, 3, 4


def _hadamard(n):
    h = np.array([[1.0]])
    while h.shape[0] < n:
        h = np.block([[h, h], [h, -h]])
    return h


_H256 = _hadamard(256) / 16.0
_H64 = _hadamard(64) / 8.0


def decode_rows(rows, fmt):
    """rows: uint8 [n, row bytes] -> float64 [n, 256] in the stored (for TQ4: rotated) coordinates."""
    if fmt == TQ4:
        import oracle
        return np.stack([oracle.decode_row(r) for r in rows]).astype(np.float64)
    from oracle import kv8
    return kv8.decode_rows(rows, fmt).astype(np.float64)


def signs():
    import oracle
    return np.array([oracle.lib().w34o_sign(i) for i in range(256)], np.float64)


def sparse_attention(k_slab, v_slab, k_fmt, v_fmt, q, gate, sel_phys, sel_logical, num_selected, seq_pos,
                     valid_token_mask, hq, hkv, sm_scale, hadamard):
    """k_slab / v_slab: uint8 [pages, hkv, 16, row bytes]; q, gate: float [T, hq, 256] (gate may be None);
    sel_phys / sel_logical: int [T, select_k]; returns float32 [T, hq, 256] (values on the fp16 grid)."""
    sg = signs()
    T = q.shape[0]
    gqa = hq // hkv
    out = np.zeros((T, hq, 256), np.float64)
    for t in range(T):
        if valid_token_mask is not None and valid_token_mask[t] == 0:
            continue
        n = min(int(num_selected[t]), sel_phys.shape[1])
        rows_k = [[] for _ in range(hkv)]
        rows_v = [[] for _ in range(hkv)]
        for i in range(n):
            pg, lg = int(sel_phys[t, i]), int(sel_logical[t, i])
            if pg < 0:
                continue
            for off in range(4):
                if 4 * lg + off > int(seq_pos[t]):
                    continue
                page, row = pg // 4, 4 * (pg % 4) + off
                for h in range(hkv):
                    rows_k[h].append(k_slab[page, h, row])
                    rows_v[h].append(v_slab[page, h, row])
        for h in range(hkv):
            if not rows_k[h]:
                continue
            kd = decode_rows(np.stack(rows_k[h]), k_fmt)
            vd = decode_rows(np.stack(rows_v[h]), v_fmt)
            for g in range(gqa):
                qh = q[t, h * gqa + g].astype(np.float64) * sm_scale
                if k_fmt == TQ4:
                    qh = _H256 @ (sg * qh)
                s = kd @ qh
                p = np.exp(s - s.max())
                o = (p @ vd) / p.sum()
                if v_fmt == TQ4:
                    o = sg * (_H256 @ o)
                out[t, h * gqa + g] = o
    if gate is not None:
        live = np.ones(T, bool) if valid_token_mask is None else np.asarray(valid_token_mask).astype(bool)
        out[live] *= 1.0 / (1.0 + np.exp(-gate.astype(np.float64)[live]))
    res = out.astype(np.float16)
    if hadamard:
        r = res.astype(np.float64).reshape(T, hq, 4, 64) @ _H64
        res = r.reshape(T, hq, 256).astype(np.float16)
    return res.astype(np.float32)
