"""Generate the golden fixtures in this folder by running the reference package itself.

Run once, on a machine that has the reference checkout (its ``src`` directory is given
with ``--ref-src``):

    python tests/golden/make_golden.py --ref-src <reference>/src

The fixtures are small ``.npz`` files holding seeded inputs and the outputs the
reference's pure-PyTorch path produced for them.  bf16 tensors are stored as their raw
int16 bit patterns (keys ending in ``_bf16``).  The test-suite never needs the reference:
it only reads these files.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-src", required=True)
    args = ap.parse_args()
    sys.path.insert(0, args.ref_src)

    from flashquant.core.codebook import _gaussian_centroids_boundaries
    from flashquant.core.compressor import KeyCompressor
    from flashquant.core.packing import nibble_pack, nibble_unpack
    from flashquant.core.quantizer import TurboQuantMSE, TurboQuantProd, haar_orthogonal
    from flashquant.kernels.attention import fused_tq_attention
    from flashquant.kernels.cpu_reference import compress_reference, decompress_reference
    from flashquant.kernels.paged_decode import split_k_paged_decode

    torch.set_num_threads(1)  # one summation order for the stored outputs

    # ---- host constants -----------------------------------------------------------
    consts = {}
    for dim, bits in [(128, 2), (128, 3), (128, 4), (64, 3), (64, 4)]:
        c, b = _gaussian_centroids_boundaries(dim, bits)
        consts[f"centroids_{dim}_{bits}"] = c.numpy()
        consts[f"boundaries_{dim}_{bits}"] = b.numpy()
    for dim, seed in [(128, 0), (128, 42), (64, 0)]:
        consts[f"rotation_{dim}_{seed}"] = haar_orthogonal(dim, seed=seed).numpy()
    consts["qjl_128_0"] = TurboQuantProd(128, 4, seed=0).qjl_matrix.numpy()
    consts["qjl_64_0"] = TurboQuantProd(64, 4, seed=0).qjl_matrix.numpy()
    np.savez_compressed(os.path.join(HERE, "constants.npz"), **consts)

    # ---- packing known answers (reference tests: tests/test_packing.py:46-64) -------
    pk = {}
    idx = torch.randint(0, 16, (5, 128), generator=torch.Generator().manual_seed(7),
                        dtype=torch.uint8)
    pk["idx"] = idx.numpy()
    pk["packed"] = nibble_pack(idx).numpy()
    pk["unpacked"] = nibble_unpack(nibble_pack(idx)).numpy()
    np.savez_compressed(os.path.join(HERE, "packing.npz"), **pk)

    # ---- quantisers (d = 128, seed 0; K with 4 outlier channels x10) ---------------
    mse = TurboQuantMSE(128, 4, seed=0)
    prod = TurboQuantProd(128, 4, seed=0)
    g = torch.Generator().manual_seed(1001)
    n_tok, n_heads = 24, 2
    v = torch.randn(n_tok, n_heads, 128, generator=g)
    k = torch.randn(n_tok, n_heads, 128, generator=g)
    outl = torch.randperm(128, generator=torch.Generator().manual_seed(1))[:4]
    k[..., outl] *= 10.0
    # adversarial rows (reference tests/test_adversarial.py): zeros, one-hot, huge, tiny
    v[0, 0] = 0.0
    v[1, 0] = 0.0
    v[1, 0, 5] = 1.0
    v[2, 0] = 1e6
    v[3, 0] = 1e-30
    v[4, 0, 17] = 1e8
    k[0, 1] = 0.0
    q = {}
    q["outlier_channels"] = outl.numpy()
    q["v"] = v.numpy()
    q["k"] = k.numpy()
    vi, vn = mse.quantize(v)
    q["v_idx"] = vi.numpy().astype(np.uint8)
    q["v_norms"] = vn.numpy()
    q["v_deq"] = mse.dequantize(vi, vn).numpy()
    vp, vn2 = compress_reference(v, mse.rotation, mse.codebook.boundaries)
    q["v_packed"] = vp.numpy()
    q["v_norms_c"] = vn2.numpy()
    q["v_decomp"] = decompress_reference(vp, vn2, mse.codebook.centroids).numpy()
    ki, kn, ks, kg = prod.quantize(k)
    q["k_idx"] = ki.numpy().astype(np.uint8)
    q["k_norms"] = kn.numpy()
    q["k_signs"] = ks.numpy().astype(np.int8)
    q["k_gamma"] = kg.numpy()
    qq = torch.randn(3, 1, 128, generator=g)
    q["ip_query"] = qq.numpy()
    q["ip_est"] = prod.estimate_inner_product(
        qq.unsqueeze(1), ki.unsqueeze(0), kn.unsqueeze(0), ks.unsqueeze(0), kg.unsqueeze(0)
    ).numpy()
    # bf16 inputs through the kernel-level reference
    vb = v.to(torch.bfloat16)
    vbp, vbn = compress_reference(vb, mse.rotation, mse.codebook.boundaries)
    q["vb_bf16"] = bf16_bits(vb)
    q["vb_packed"] = vbp.numpy()
    q["vb_norms"] = vbn.numpy()
    np.savez_compressed(os.path.join(HERE, "quantize.npz"), **q)

    # ---- KeyCompressor scores (reference core/compressor.py:151-192) ----------------
    kc = KeyCompressor(128, 4, seed=0)
    keys = torch.randn(1, 2, 9, 128, generator=g)
    qry = torch.randn(1, 2, 3, 128, generator=g)
    comp = kc.compress(keys)
    sc = kc.asymmetric_attention_scores(qry, comp)
    np.savez_compressed(
        os.path.join(HERE, "key_scores.npz"),
        keys=keys.numpy(), query=qry.numpy(), scores=sc.numpy(),
    )

    # ---- paged decode (small; both codebooks differ: K 3-bit, V 4-bit) ---------------
    h_kv, h_q, d, bs = 2, 8, 128, 16
    lens = [0, 1, 15, 16, 17, 53]
    max_blocks = 4
    nb = 32
    g = torch.Generator().manual_seed(1002)
    cache = torch.zeros(nb, bs, h_kv * (d + 8), dtype=torch.uint8)
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(2))
    bt = perm[: len(lens) * max_blocks].reshape(len(lens), max_blocks).int()
    k_all = torch.randn(len(lens), 64, h_kv, d, generator=g)
    k_all[..., outl] *= 10.0
    v_all = torch.randn(len(lens), 64, h_kv, d, generator=g)
    rot = mse.rotation
    ck, bk = prod.mse_quantizer.codebook.centroids, prod.mse_quantizer.codebook.boundaries
    cv, bv = mse.codebook.centroids, mse.codebook.boundaries
    flat = cache.view(-1, h_kv * (d + 8))
    for i, n in enumerate(lens):
        if n == 0:
            continue
        kp, kn_ = compress_reference(k_all[i, :n], rot, bk)
        vp_, vn_ = compress_reference(v_all[i, :n], rot, bv)
        row = torch.empty(n, h_kv * (d + 8), dtype=torch.uint8)
        a = h_kv * d // 2
        row[:, :a] = kp.reshape(n, -1)
        row[:, a:a + 4 * h_kv] = kn_.reshape(n, h_kv).contiguous().view(torch.uint8)
        row[:, a + 4 * h_kv:2 * a + 4 * h_kv] = vp_.reshape(n, -1)
        row[:, 2 * a + 4 * h_kv:] = vn_.reshape(n, h_kv).contiguous().view(torch.uint8)
        t = torch.arange(n)
        slots = bt[i][t // bs].long() * bs + t % bs
        flat[slots] = row
    qd = torch.randn(len(lens), h_q, d, generator=g).to(torch.bfloat16)
    out = split_k_paged_decode(qd, cache, bt, torch.tensor(lens, dtype=torch.int32),
                               ck, cv, rot, h_kv, d, bs)
    qd16 = qd.to(torch.float16)
    out16 = split_k_paged_decode(qd16, cache, bt, torch.tensor(lens, dtype=torch.int32),
                                 ck, cv, rot, h_kv, d, bs, sm_scale=0.05)
    np.savez_compressed(
        os.path.join(HERE, "paged_decode.npz"),
        kv_cache=cache.numpy(), block_table=bt.numpy(),
        seq_lens=np.array(lens, dtype=np.int32), q_bf16=bf16_bits(qd), out_bf16=bf16_bits(out),
        q_f16=qd16.numpy(), out_f16=out16.numpy(), sm_scale_f16=np.float32(0.05),
        h_kv=h_kv, h_q=h_q, d=d, block_size=bs,
    )

    # ---- fused prefill attention (small) ---------------------------------------------
    g = torch.Generator().manual_seed(1003)
    b_, hq_, hkv_, n_ = 2, 4, 2, 80
    qa = torch.randn(b_, hq_, n_, d, generator=g).to(torch.bfloat16)
    ka = torch.randn(b_, hkv_, n_, d, generator=g)
    ka[..., outl] *= 10.0
    va = torch.randn(b_, hkv_, n_, d, generator=g)
    kp, kn_ = compress_reference(ka.reshape(b_ * hkv_, n_, d).to(torch.bfloat16), rot, bk)
    vp_, vn_ = compress_reference(va.reshape(b_ * hkv_, n_, d).to(torch.bfloat16), rot, bv)
    kp = kp.reshape(b_, hkv_, n_, d // 2)
    kn_ = kn_.reshape(b_, hkv_, n_, 1)
    vp_ = vp_.reshape(b_, hkv_, n_, d // 2)
    vn_ = vn_.reshape(b_, hkv_, n_, 1)
    oc = fused_tq_attention(qa, kp, kn_, vp_, vn_, ck, cv, rot, is_causal=True)
    on = fused_tq_attention(qa, kp, kn_, vp_, vn_, ck, cv, rot, is_causal=False)
    np.savez_compressed(
        os.path.join(HERE, "prefill.npz"),
        q_bf16=bf16_bits(qa), k_packed=kp.numpy(), k_norms=kn_.numpy(),
        v_packed=vp_.numpy(), v_norms=vn_.numpy(),
        out_causal_bf16=bf16_bits(oc), out_full_bf16=bf16_bits(on),
    )
    # ---- CompressedDynamicCache on a stand-in for DynamicCache ----------------------------
    from flashquant.cache.hf_cache import CompressedDynamicCache

    class Layer:
        def __init__(self):
            self.keys = self.values = None
            self.is_initialized = False

        def lazy_initialization(self, _):
            self.is_initialized = True

    class Cache:
        def __init__(self):
            self.layers = []
            self.layer_class_to_replicate = Layer

        def update(self, k_, v_, layer_idx, cache_kwargs=None):
            return k_, v_

        def get_seq_length(self, layer_idx=0):
            return 0

    g = torch.Generator().manual_seed(1004)
    wrapped = CompressedDynamicCache(Cache(), head_dim=d, bits=4, max_seq_len=64)
    hc = {"rotation_k": wrapped.rotation_k.numpy(), "rotation_v": wrapped.rotation_v.numpy()}
    steps = [20, 1, 3, 1]
    for layer in (0, 1):
        for i, s_new in enumerate(steps):
            kx = torch.randn(2, 2, s_new, d, generator=g)
            kx[..., outl] *= 10.0
            vx = torch.randn(2, 2, s_new, d, generator=g)
            kx, vx = kx.to(torch.bfloat16), vx.to(torch.bfloat16)
            ko, vo = wrapped.cache.update(kx, vx, layer)
            hc[f"k_in_{layer}_{i}_bf16"] = bf16_bits(kx)
            hc[f"v_in_{layer}_{i}_bf16"] = bf16_bits(vx)
        kp, kn_, vp_, vn_ = wrapped.get_compressed(layer)
        hc[f"k_packed_{layer}"] = kp.contiguous().numpy()
        hc[f"k_norms_{layer}"] = kn_.contiguous().numpy()
        hc[f"v_packed_{layer}"] = vp_.contiguous().numpy()
        hc[f"v_norms_{layer}"] = vn_.contiguous().numpy()
        hc[f"k_out_{layer}_bf16"] = bf16_bits(ko)
        hc[f"v_out_{layer}_bf16"] = bf16_bits(vo)
        hc[f"seq_len_{layer}"] = np.int64(wrapped.cache.get_seq_length(layer))
    hc["steps"] = np.array(steps, dtype=np.int64)
    hc["vram_bytes"] = np.int64(wrapped.vram_bytes())
    hc["compressed_vram_bytes"] = np.int64(wrapped.compressed_vram_bytes())
    hc["baseline_vram_bytes"] = np.int64(wrapped.baseline_vram_bytes())
    wrapped.restore()
    np.savez_compressed(os.path.join(HERE, "hf_cache.npz"), **hc)

    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
