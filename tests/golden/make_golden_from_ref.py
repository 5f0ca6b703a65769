"""Generates the golden fixtures from the reference's own CUDA kernels.

Run on a machine with a GPU and ``oracle/_ref/ref_kernels.so`` (the reference's
``bsi_cuda_kernels.cu`` compiled unmodified for sm_100a by ``oracle/build.py``):

    python tests/golden/make_golden_from_ref.py <output-dir>

It writes ``ref_fixed76.npz``: seeded inputs plus what the reference kernels produced for them --
packed query/key words, shifts and scales, clamped key integers, EWAH streams, and fixed76
chunk-scale dot outputs -- and ``ref_modes.npz`` with the other modes of the path: the variable-slice
mode (int64 rounding + ballot packer, generic float-weight dot kernels), the fixed-bit row-scale dot
(word counts that rule out chunk scales) and packing with outlier clipping. The CPU checker (``oracle/``) and the CUDA library are both tested
against this file. Inputs are synthetic (shapes and value distributions of the benchmark
configurations, scaled down); nothing here comes from an evaluation dataset.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import _inputs  # noqa: E402
from oracle import ref_gpu  # noqa: E402


def u64(t):
    return t.detach().cpu().numpy().view(np.uint64)


def structured_words(S, W, seed):
    rng = np.random.default_rng(seed)
    ones = np.uint64(0xFFFFFFFFFFFFFFFF)
    w = rng.integers(1, 2 ** 63, (S, W), dtype=np.uint64)
    for s in range(S):
        k = s % 6
        if k == 0:
            w[s] = 0
        elif k == 1:
            w[s] = ones
        elif k == 2:
            w[s][rng.random(W) < 0.7] = 0
        elif k == 3:
            w[s][rng.random(W) < 0.5] = 0
            w[s][rng.random(W) < 0.4] = ones
        elif k == 4:
            w[s] = 0
            w[s][rng.integers(0, W)] = 1
    return w


def main(outdir):
    assert ref_gpu.available(), "needs a GPU and oracle/_ref/ref_kernels.so"
    dev = "cuda"
    out = {}
    si = np.float32(1.0 / 10.0 ** 4)

    # dot cases: (name, queries, keys); Q and R multiples of 32 so that the fixed76 kernels are selected
    cases = {
        "c1": _inputs.c1(Q=32, R=32, D=512),
        "fc1": _inputs.fc1(Q=32, R=160, D=1024),            # 160 = 128 (rsweep4) + 32 (tail kernel)
        "fc2": _inputs.fc2(Q=32, R=32, D=2048),
    }
    for name, (q, k) in cases.items():
        k = k.half().float()     # keys rounded to fp16-representable values: half the fixture size, still fp32 input
        qd, kd = q.to(dev), k.to(dev)
        qw, qsh, qsc = ref_gpu.pack_queries_chunk(qd, 2, 7)
        kw, ksh, ksc, kint = ref_gpu.pack_rows(kd, 2, 6)
        Bw = ref_gpu.slice_weights(6, k.shape[0], dev, ksc)
        o = ref_gpu.dot_fixed76(qw, qsc, kw, Bw, si)
        torch.cuda.synchronize()
        out[f"{name}_q"] = q.numpy() if q.dtype == torch.float32 else q.view(torch.int16).numpy()
        out[f"{name}_q_dtype"] = np.array(str(q.dtype))
        out[f"{name}_k_f16bits"] = k.half().view(torch.int16).numpy()
        out[f"{name}_q_words"] = u64(qw)
        out[f"{name}_q_shifts"] = qsh.cpu().numpy()
        out[f"{name}_q_scales"] = qsc.cpu().numpy()
        out[f"{name}_k_words"] = u64(kw)
        out[f"{name}_k_shifts"] = ksh.cpu().numpy()
        out[f"{name}_k_scales"] = ksc.cpu().numpy()
        out[f"{name}_k_ints"] = kint.cpu().numpy().astype(np.int8)
        out[f"{name}_Bw"] = Bw.cpu().numpy()
        out[f"{name}_out"] = o.cpu().numpy()
        # EWAH of the query slices at the benchmark's threshold
        st, off, ln, fl, cnt = ref_gpu.ewah_encode(qw.view(-1, qw.shape[2]), 0.5)
        out[f"{name}_ewah_stream"] = u64(st)
        out[f"{name}_ewah_off"] = off.cpu().numpy()
        out[f"{name}_ewah_len"] = ln.cpu().numpy()
        out[f"{name}_ewah_flags"] = fl.cpu().numpy()
        out[f"{name}_ewah_counts"] = u64(cnt)

    # pack-only cases
    for dtype, tag in [(torch.float32, "f32"), (torch.float16, "f16"), (torch.bfloat16, "bf16")]:
        x = _inputs.edge_rows(512, dtype)
        w, sh, sc = ref_gpu.pack_queries_chunk(x.to(dev), 2, 7)
        out[f"edge_{tag}_x"] = x.float().numpy()
        out[f"edge_{tag}_words"] = u64(w)
        out[f"edge_{tag}_shifts"] = sh.cpu().numpy()
        kw, ksh, ksc, kint = ref_gpu.pack_rows(x.float().to(dev), 2, 6)
        out[f"edge_{tag}_row_words"] = u64(kw)
        out[f"edge_{tag}_row_shifts"] = ksh.cpu().numpy()
    q16, _ = _inputs.fc1(Q=8, R=8, D=1024, dtype=torch.bfloat16)
    w, sh, sc = ref_gpu.pack_queries_chunk(q16.to(dev), 2, 7)
    out["bf16_x"] = q16.float().numpy()
    out["bf16_words"] = u64(w)
    out["bf16_shifts"] = sh.cpu().numpy()

    # EWAH on structured words, several thresholds, plus decode
    for W in (5, 33, 128):
        words = structured_words(18, W, W)
        wt = torch.from_numpy(words.view(np.int64)).to(dev)
        out[f"ewah{W}_words"] = words
        for thr in (0.5, 0.2, 1.0):
            st, off, ln, fl, cnt = ref_gpu.ewah_encode(wt, thr)
            tag = f"ewah{W}_t{int(thr * 10)}"
            out[f"{tag}_stream"] = u64(st)
            out[f"{tag}_off"] = off.cpu().numpy()
            out[f"{tag}_len"] = ln.cpu().numpy()
            out[f"{tag}_flags"] = fl.cpu().numpy()
            back = ref_gpu.ewah_decode(st, off, ln, W)
            assert np.array_equal(u64(back), words)
    torch.cuda.synchronize()
    os.makedirs(outdir, exist_ok=True)
    path = os.path.join(outdir, "ref_fixed76.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


def bit_length(v):
    return int(v).bit_length()


def modes(outdir):
    """Variable-slice mode, row-scale dot, outlier clipping: what the reference kernels give for them."""
    assert ref_gpu.available(), "needs a GPU and oracle/_ref/ref_kernels.so"
    dev = "cuda"
    out = {}
    si = np.float32(1.0 / 10.0 ** 4)

    # variable-slice mode (bsi_vector_cuda.cpp:746-754): slice count = bit_width(max |v|) + 2, at least 2; queries
    # per batch, keys here at the widest row's count (a narrower row sign-extends to it)
    q, k = _inputs.c1(Q=32, R=64, D=512)
    k = k.half().float()
    qd, kd = q.to(dev), k.to(dev)
    _, qi = ref_gpu.pack_plain(qd, 2, 2)
    _, ki = ref_gpu.pack_plain(kd, 2, 2)
    Sq = max(2, bit_length(qi.abs().max().item()) + 2)
    Sk = max(2, bit_length(ki.abs().max().item()) + 2)
    qw, _ = ref_gpu.pack_plain(qd, 2, Sq)
    kw, _ = ref_gpu.pack_plain(kd, 2, Sk)
    Aw = ref_gpu.slice_weights(Sq, 32, dev)
    Bw = ref_gpu.slice_weights(Sk, 64, dev)
    out["var_q"] = q.numpy()
    out["var_k_f16bits"] = k.half().view(torch.int16).numpy()
    out["var_q_ints"] = qi.cpu().numpy().astype(np.int32)
    out["var_k_ints"] = ki.cpu().numpy().astype(np.int32)
    out["var_q_words"] = u64(qw)
    out["var_k_words"] = u64(kw)
    out["var_out_tc"] = ref_gpu.dot_generic(qw, Aw, kw, Bw, si, tensor_core=True).cpu().numpy()
    out["var_out_plain"] = ref_gpu.dot_generic(qw, Aw, kw, Bw, si, tensor_core=False).cpu().numpy()

    # fixed-bit mode with one scale per query row: BSI_FIXED_CHUNK_SCALE=0 ("row", 8 words per slice, tensor-core
    # and plain generic kernels) and a word count that rules chunk scales out ("rowr", 5 words per slice:
    # bsi_vector_cuda.cpp:980-994; the dispatcher then takes the plain kernel whatever the switch says)
    for tag, D in (("row", 512), ("rowr", 320)):
        q, k = _inputs.fc1(Q=32, R=32, D=D, dtype=torch.float32)
        k = k.half().float()
        qd, kd = q.to(dev), k.to(dev)
        qw, qsh, qsc, qint = ref_gpu.pack_rows(qd, 2, 7)
        kw, ksh, ksc, kint = ref_gpu.pack_rows(kd, 2, 6)
        Aw = ref_gpu.slice_weights(7, 32, dev, qsc)
        Bw = ref_gpu.slice_weights(6, 32, dev, ksc)
        out[f"{tag}_q"] = q.numpy()
        out[f"{tag}_k_f16bits"] = k.half().view(torch.int16).numpy()
        out[f"{tag}_q_words"] = u64(qw)
        out[f"{tag}_q_scales"] = qsc.cpu().numpy()
        out[f"{tag}_k_words"] = u64(kw)
        out[f"{tag}_k_scales"] = ksc.cpu().numpy()
        out[f"{tag}_out_tc"] = ref_gpu.dot_generic(qw, Aw, kw, Bw, si, tensor_core=True).cpu().numpy()
        out[f"{tag}_out_plain"] = ref_gpu.dot_generic(qw, Aw, kw, Bw, si, tensor_core=False).cpu().numpy()

    # outlier clipping (BSI_FIXED_CLIP_K = 3)
    x, kx = _inputs.fc1(Q=16, R=16, D=1000, dtype=torch.float16)
    w, sh, sc = ref_gpu.pack_queries_chunk(x.to(dev), 2, 7, clip_k=3.0)
    out["clip_x_f16bits"] = x.view(torch.int16).numpy()
    out["clip_words"] = u64(w)
    out["clip_shifts"] = sh.cpu().numpy()
    kx = kx.half().float()
    kw, ksh, ksc, kint = ref_gpu.pack_rows(kx.to(dev), 2, 6, clip_k=3.0)
    out["clip_k_f16bits"] = kx.half().view(torch.int16).numpy()
    out["clip_row_words"] = u64(kw)
    out["clip_row_shifts"] = ksh.cpu().numpy()
    out["clip_row_ints"] = kint.cpu().numpy().astype(np.int8)
    torch.cuda.synchronize()
    os.makedirs(outdir, exist_ok=True)
    path = os.path.join(outdir, "ref_modes.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    target = sys.argv[1] if len(sys.argv) > 1 else HERE
    main(target)
    modes(target)
