"""Writes a fa_data.h with the array names, shapes and macro set of the reference's generator
(kernels/flash_attention_mx_gqa/fa_gen_data.py:122-158), from seeded inputs quantized by the CPU oracle.

Layouts as the reference emits them:
  QK_A_in            [NQ*SQ][D]          Q codes per query head
  QK_A_scales_row    [NQ*GK][SQ]         Q scales, group-major per head
  QK_B_blocks        [NKV*NBU*D][BK]     K^T per KV head and key block
  QK_B_scales_blocks [NKV*NBU*GK][BK]
  V_in               [NKV*NBU*BK][D]     V per KV head, blocks of 32 along the keys
  V_scales           [NKV*NBU*GKB][D]
  O_gold             [NQ*SQ][D]          bf16 codes: here the CPU oracle's output at the kernel's block_n
Test infrastructure: imports the oracle."""
import numpy as np

import oracle


def _rows(mat, fmt):
    return ",\n".join("    { " + ", ".join(fmt % int(v) for v in row) + " }" for row in mat)


def blocks_used(Sq, Sk, q_pos0, Bk):
    """Leading key blocks not wholly above the diagonal (flash_attention_model.py:182-186)."""
    return min(Sk // Bk, (q_pos0 + Sq - 1) // Bk + 1)


def write_fa_data(path, *, Sq=64, Sk=256, d=64, n_q=8, n_kv=2, q_pos0=64, Bk=64, seed=0, block_n=128):
    rng = np.random.default_rng(seed)
    Q = rng.standard_normal((n_q, Sq, d)).astype(np.float32)
    K = rng.standard_normal((n_kv, Sk, d)).astype(np.float32)
    V = rng.standard_normal((n_kv, Sk, d)).astype(np.float32)
    GK, GKB, nbu = d // 32, Bk // 32, blocks_used(Sq, Sk, q_pos0, Bk)
    skv = nbu * Bk
    scale = float(np.float32(1.0 / np.sqrt(d)))
    scale_bf16 = oracle.lib().rko_f32_to_bf16(scale)
    scale_used = float(np.array([scale_bf16 << 16], np.uint32).view(np.float32)[0])

    qc, qs, kc, ks, vc, vs = [], [], [], [], [], []
    for h in range(n_q):
        c, s = oracle.quantize(Q[h], axis=-1)
        qc.append(c); qs.append(s)
    for kv in range(n_kv):
        c, s = oracle.quantize(K[kv, :skv], axis=-1)
        kc.append(c); ks.append(s)
        c, s = oracle.quantize(V[kv, :skv], axis=0)        # V: blocks along the keys (gen_data.py:77)
        vc.append(c); vs.append(s)
    A_in = np.concatenate(qc, 0)                                            # [NQ*SQ][D]
    A_scales_row = np.concatenate([s.T for s in qs], 0)                     # [NQ*GK][SQ]
    B_blocks = np.concatenate([kc[kv][j * Bk:(j + 1) * Bk].T for kv in range(n_kv) for j in range(nbu)], 0)
    B_scales = np.concatenate([ks[kv][j * Bk:(j + 1) * Bk].T for kv in range(n_kv) for j in range(nbu)], 0)
    V_in = np.concatenate(vc, 0)                                            # [NKV*NBU*BK][D]
    V_scales = np.concatenate(vs, 0)                                        # [NKV*NBU*GKB][D]

    ref = oracle.attn_prefill(np.stack(qc)[None], np.stack(kc)[None], np.stack(vc)[None], np.stack(qs)[None],
                              np.stack(ks)[None], np.stack(vs)[None], causal=True, softmax_scale=scale_used,
                              q_pos0=q_pos0, v_scale_axis=0, block_n=block_n)
    O_gold = ref["o_bf16"][0].reshape(n_q * Sq, d)

    with open(path, "w") as f:
        f.write("#ifndef FA_DATA_H\n#define FA_DATA_H\n\n#include <stdint.h>\n\n")
        f.write(f"#define FA_SQ {Sq}\n#define FA_SK {Sk}\n#define FA_D {d}\n#define FA_GK {GK}\n#define FA_GKV {Sk // 32}\n")
        f.write(f"#define FA_BK {Bk}\n#define FA_NBLK {Sk // Bk}\n#define FA_GKB {GKB}\n")
        f.write(f"#define FA_NQ {n_q}\n#define FA_NKV {n_kv}\n#define FA_GRP {n_q // n_kv}\n#define FA_QPOS0 {q_pos0}\n")
        f.write(f"#define FA_NBLK_USED {nbu}\n#define FA_SOFTMAX_SCALE_BF16 0x{scale_bf16:04x}\n\n")
        f.write(f"static const uint8_t QK_A_in[FA_NQ*FA_SQ][FA_D] = {{\n{_rows(A_in, '0x%02x')}\n}};\n\n")
        f.write(f"static const uint8_t QK_A_scales_row[FA_NQ*FA_GK][FA_SQ] = {{\n{_rows(A_scales_row, '0x%02x')}\n}};\n\n")
        f.write(f"static const uint8_t QK_B_blocks[FA_NKV*FA_NBLK_USED*FA_D][FA_BK] = {{\n{_rows(B_blocks, '0x%02x')}\n}};\n\n")
        f.write(f"static const uint8_t QK_B_scales_blocks[FA_NKV*FA_NBLK_USED*FA_GK][FA_BK] = {{\n{_rows(B_scales, '0x%02x')}\n}};\n\n")
        f.write(f"static const uint8_t V_in[FA_NKV*FA_NBLK_USED*FA_BK][FA_D] = {{\n{_rows(V_in, '0x%02x')}\n}};\n\n")
        f.write(f"static const uint8_t V_scales[FA_NKV*FA_NBLK_USED*FA_GKB][FA_D] = {{\n{_rows(V_scales, '0x%02x')}\n}};\n\n")
        f.write(f"static const uint16_t O_gold[FA_NQ*FA_SQ][FA_D] = {{\n{_rows(O_gold, '0x%04x')}\n}};\n\n")
        f.write("#endif // FA_DATA_H\n")
    return dict(A_in=A_in, A_scales_row=A_scales_row, B_blocks=B_blocks, B_scales=B_scales, V_in=V_in,
                V_scales=V_scales, O_gold=O_gold, nbu=nbu, kc=kc, ks=ks)
