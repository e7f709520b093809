"""bfuse_default_launch without a device (context NULL = 148 SMs): the tilings the runtime picks for
the tensor-core operators -- tile width / height, k-slices, ring depth, conv pixel-tile width."""
import bfuse_project_b200 as bf


def default(op, shape):
    d = bf.KernelDesc()
    d.KernelName = b"k"
    d.op = op
    for i, v in enumerate(shape):
        d.shape[i] = v
    rc = bf.lib().bfuse_default_launch(None, d)
    assert rc == 0, rc
    return d


def gemm(op, batch, m, n, k, **kw):
    d = default(op, (batch, m, n, k, kw.get("bn", 0), kw.get("split", 0), kw.get("bm", 0)))
    return {"grid": d.GridDim.tuple(), "bn": d.shape[4], "split": d.shape[5], "bm": d.shape[6], "smem": d.smem_bytes}


def test_projection_pairs_get_narrow_unsplit_tiles_and_a_whole_sm_ring():
    q = gemm(bf.OP_GEMM_TF32, 1, 512, 768, 768)           # BERT Q / K projection
    assert (q["bn"], q["split"], q["bm"], q["grid"]) == (64, 1, 128, (4, 12, 1))
    assert q["smem"] == 2048 + 8 * (128 + 64) * 128        # 48 CTAs and an equal partner: every CTA has an SM
    kv = gemm(bf.OP_GEMM_BF16, 1, 512, 1024, 4096)         # Llama k / v projection
    assert (kv["bn"], kv["split"], kv["grid"]) == (64, 1, (4, 16, 1)) and kv["smem"] == 2048 + 8 * 192 * 128


def test_large_long_k_gemm_gets_tall_tiles():
    g = gemm(bf.OP_GEMM_BF16, 1, 512, 14336, 4096)         # Llama gate / up projection
    assert (g["bn"], g["split"], g["bm"], g["grid"]) == (256, 1, 256, (2, 56, 1))
    assert g["smem"] == 2048 + 3 * 512 * 128
    s = gemm(bf.OP_GEMM_TF32, 1024, 512, 512, 64)          # many tiles but two K blocks: bound by its stores
    assert s["bm"] == 128


def test_skinny_long_k_gemm_is_split_over_a_cluster():
    g = gemm(bf.OP_GEMM_BF16, 1, 128, 128, 8192)
    assert g["split"] > 1 and g["grid"][0] == g["split"]
    assert gemm(bf.OP_GEMM_BF16, 1, 128, 128, 8192, split=1)["split"] == 1   # a fixed value is kept


def test_explicit_tile_fields_are_validated():
    d = bf.KernelDesc()
    d.KernelName, d.op = b"k", bf.OP_GEMM_TF32
    for i, v in enumerate((1, 512, 512, 512, 48, 1, 0)):
        d.shape[i] = v
    assert bf.lib().bfuse_default_launch(None, d) == 2       # BN must be 32, 64, 128 or 256
    for i, v in enumerate((1, 512, 512, 512, 256, 2, 256)):
        d.shape[i] = v
    assert bf.lib().bfuse_default_launch(None, d) == 2       # tall tiles only unsplit


def test_conv_pixel_tile_width_and_k_slices_follow_the_image_count():
    one = default(bf.OP_CONV2D_TF32, (1, 64, 56, 56, 128, 3, 3, 2, 1))        # 784 pixels of one image, 18 K blocks
    assert (one.shape[9], one.shape[10]) == (32, 4) and one.GridDim.tuple() == (100, 1, 1)
    short = default(bf.OP_CONV2D_TF32, (1, 64, 56, 56, 128, 1, 1, 2, 0))      # K = 64: nothing to split
    assert (short.shape[9], short.shape[10]) == (32, 1) and short.GridDim.tuple() == (25, 1, 1)
    many = default(bf.OP_CONV2D_TF32, (256, 64, 56, 56, 128, 3, 3, 2, 1))
    # 1792 tiles, staged: more than the two CTAs per SM that fit at a time, so a CTA takes 6 or 7 tiles (every 296th)
    assert (many.shape[9], many.shape[10], many.shape[11]) == (128, 1, 1) and many.GridDim.tuple() == (296, 1, 1)
    some = default(bf.OP_CONV2D_TF32, (32, 64, 56, 56, 128, 3, 3, 2, 1))      # 224 tiles: one each
    assert (some.shape[9], some.shape[11]) == (128, 1) and some.GridDim.tuple() == (7, 1, 32)
    deep = default(bf.OP_CONV2D_TF32, (1, 512, 7, 7, 512, 3, 3, 1, 1))        # K = 4608 on 8 tiles: the table takes 36 KB
    assert (deep.shape[9], deep.shape[10]) == (32, 4) and deep.GridDim.tuple() == (8, 4, 1)
    assert deep.smem_bytes >= 2048 + 36 * 1024 + 4 * 16 * 1024 + 16 * 1024   # header, table, 4 partial sums, store buffers


def test_automatic_k_slices_are_one_or_four():
    """Any two operators the runtime tiled itself can share a launch: their cluster widths are 1 or 4."""
    seen = set()
    for m, n, k in ((128, 128, 8192), (256, 256, 4096), (512, 768, 768), (64, 64, 16384), (128, 512, 2048), (512, 512, 64)):
        seen.add(gemm(bf.OP_GEMM_BF16, 1, m, n, k)["split"])
    for sh in ((1, 256, 14, 14, 256, 3, 3, 1, 1), (1, 128, 28, 28, 128, 3, 3, 1, 1), (1, 768, 17, 17, 192, 1, 1, 1, 0), (4, 64, 56, 56, 64, 3, 3, 1, 1)):
        seen.add(default(bf.OP_CONV2D_TF32, sh).shape[10])
    assert seen <= {1, 4} and 4 in seen


def test_share_hint_budgets_the_sms_per_co_runner():
    """BFUSE_FLAG_SHARE(n): the operator is tiled for 1 / n of the SMs (absent: a pair, n = 2)."""
    def g(op, shape, share):
        d = bf.KernelDesc()
        d.KernelName, d.op, d.flags = b"k", op, bf.flag_share(share) if share else 0
        for i, v in enumerate(shape):
            d.shape[i] = v
        assert bf.lib().bfuse_default_launch(None, d) == 0
        return d.GridDim.tuple(), d.shape[4], d.shape[5], d.shape[6]
    q = (1, 512, 4096, 4096, 0, 0, 0)                                  # Llama q projection, bf16
    assert g(bf.OP_GEMM_BF16, q, 0) == g(bf.OP_GEMM_BF16, q, 2)        # no hint = a pair
    assert g(bf.OP_GEMM_BF16, q, 1) == ((4, 32, 1), 128, 1, 128)       # alone: 128 CTAs of 128 x 128
    assert g(bf.OP_GEMM_BF16, q, 2) == ((4, 16, 1), 256, 1, 128)
    assert g(bf.OP_GEMM_BF16, q, 3) == ((4, 16, 1), 256, 1, 128)       # a third of the SMs: still 128-row tiles (no second wave to save)
    gate = (1, 512, 14336, 4096, 0, 0, 0)
    assert g(bf.OP_GEMM_BF16, gate, 1) == ((2, 56, 1), 256, 1, 256)    # alone, 224 tiles = 2 waves: 256-row tiles make it one
    assert g(bf.OP_GEMM_BF16, gate, 2) == ((2, 56, 1), 256, 1, 256)
    ffn2 = (1, 512, 768, 3072, 0, 0, 0)                                # BERT FFN down projection, tf32: long K, few tiles
    assert g(bf.OP_GEMM_TF32, ffn2, 1)[2] == 4 and g(bf.OP_GEMM_TF32, ffn2, 4)[2] == 1   # k-slices only while SMs are idle
    conv = (1, 64, 56, 56, 128, 3, 3, 2, 1)                            # 784 pixels, 18 K blocks
    d = bf.KernelDesc()
    d.KernelName, d.op, d.flags = b"k", bf.OP_CONV2D_TF32, bf.flag_share(4)
    for i, v in enumerate(conv):
        d.shape[i] = v
    assert bf.lib().bfuse_default_launch(None, d) == 0 and d.shape[10] == 1 and d.shape[9] == 32   # a quarter of the SMs: 25 tiles fill it unsplit


def test_lone_long_k_gemm_may_take_two_k_slices():
    """An operator that runs alone (share 1) may split a very long K in two; operators that share a launch keep 1 or 4."""
    def split(op, shape, share):
        d = bf.KernelDesc()
        d.KernelName, d.op, d.flags = b"k", op, bf.flag_share(share)
        for i, v in enumerate(shape):
            d.shape[i] = v
        assert bf.lib().bfuse_default_launch(None, d) == 0
        return d.shape[5]
    down = (1, 512, 4096, 14336, 0, 0, 0)                       # Llama down projection: 224 K blocks in bf16
    assert split(bf.OP_GEMM_BF16, down, 1) == 2 and split(bf.OP_GEMM_BF16, down, 2) in (1, 4)
    assert split(bf.OP_GEMM_TF32, (1, 512, 4096, 4096, 0, 0, 0), 1) == 1      # 128 K blocks: unsplit is as fast
