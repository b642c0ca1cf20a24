"""Small Dabilorn configurations for the tests: other sizes, orders, chunk sizes and constants than any model folder that is served."""


def yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=1e4, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
        if scaling is not None:
            m["rot"]["scaling"] = scaling
    return m


def attn(heads, kv_heads, dim, vdim, scale, chunk=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = rot
    return m


def wkv(heads, dim, decay_rank):
    return {"heads": heads, "dim": dim, "decay_rank": decay_rank}


def moe(experts, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(vocab, width, eps, taps, layers):
    cfg = {"architecture": "Dabilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if taps is not None:
        cfg["canon"] = {"taps": taps}
    return cfg


# every mixer; grouped kv heads; a chunk that is a multiple of nothing; part of a head rotated; value sizes above and below the
# key size; several experts per token; a layer without a feed-forward and one without a shared expert; rescaled frequencies whose
# ramp lies inside the pairs
DAB_A = model(131, 64, 1e-5, 3, [
    layer("attention", attn(4, 2, 16, 24, 0.3, chunk=11, rot={"base": 100.0, "dims": 8}), moe(5, 2, 40, shared=24)),
    layer("wkv", wkv(2, 16, 8), moe(3, 3, 24)),
    layer("latent_attention", latent(3, 12, 8, 20, 24, 40, 0.2, base=50.0, scaling=yarn(4.0, 64, 8.0, 1.0))),
    layer("attention", attn(2, 1, 24, 8, 0.25, chunk=32, rot={"base": 1e4, "dims": 24}), moe(5, 2, 40, shared=24)),
    layer("latent_attention", latent(2, 16, 4, 16, 20, 12, 0.3, base=1e3), moe(6, 1, 16, shared=8))])

# sizes that are multiples of nothing; one kv head per head; a chunk of one position; one tap (no state) ; no rescaling; a
# rotated part of two values; a query latent wider than the model
DAB_B = model(97, 50, 3e-4, 1, [
    layer("latent_attention", latent(3, 10, 2, 14, 18, 60, 0.4, base=30.0), moe(4, 1, 30, shared=10)),
    layer("attention", attn(3, 3, 10, 10, 0.4, chunk=1, rot={"base": 30.0, "dims": 10}), moe(2, 2, 18)),
    layer("wkv", wkv(3, 12, 5)),
    layer("attention", attn(2, 1, 12, 6, 0.25, chunk=8, rot={"base": 1e6, "dims": 2}), moe(4, 1, 30, shared=10)),
    layer("latent_attention", latent(1, 6, 6, 6, 10, 4, 0.5, base=10.0, scaling=yarn(8.0, 32, 4.0, 0.5)))])

# head sizes the tensor-core attention kernels take (64 and 128 values), a chunk of several pages and one that no page edge
# meets, five taps, a latent row of 128 values
DAB_C = model(120, 128, 1e-6, 5, [
    layer("attention", attn(8, 2, 64, 64, 0.125, chunk=32, rot={"base": 1000.0, "dims": 16}), moe(8, 2, 64, shared=32)),
    layer("latent_attention", latent(4, 32, 24, 32, 104, 64, 0.12, base=1e5, scaling=yarn(2.0, 128, 16.0, 2.0)), moe(8, 2, 64, shared=32)),
    layer("wkv", wkv(2, 64, 16), moe(6, 4, 32)),
    layer("attention", attn(2, 2, 128, 128, 0.09, chunk=70, rot={"base": 500.0, "dims": 128}))])

# no convolution in front of the mixers; an attention layer without a mask and without a rotation (every earlier key weighs in);
# a latent without a rotated part; every expert chosen; two taps elsewhere are covered by E
DAB_D = model(80, 40, 1e-5, None, [
    layer("wkv", wkv(2, 20, 4), moe(2, 2, 16, shared=16)),
    layer("attention", attn(2, 2, 20, 20, 0.2), moe(3, 2, 44)),
    layer("latent_attention", latent(5, 8, 0, 8, 16, 16, 0.35), moe(1, 1, 16, shared=4)),
    layer("attention", attn(1, 1, 40, 12, 0.15, chunk=3))])

# two taps; the layers in an order that opens with attention; a chunk longer than every request
DAB_E = model(64, 48, 1e-5, 2, [
    layer("attention", attn(3, 1, 16, 16, 0.25, chunk=500, rot={"base": 250.0, "dims": 4}), moe(4, 1, 24, shared=24)),
    layer("latent_attention", latent(2, 8, 8, 12, 16, 24, 0.3, base=2e4, scaling=yarn(2.0, 16, 2.0, 1.0)), moe(4, 1, 24, shared=24)),
    layer("wkv", wkv(3, 16, 6), moe(4, 1, 24, shared=24))])

ALL = {"A": DAB_A, "B": DAB_B, "C": DAB_C, "D": DAB_D, "E": DAB_E}
