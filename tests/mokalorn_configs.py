"""Small Mokalorn configurations for the tests: other sizes, orders, chunk sizes and constants than any model folder that is served."""


def attn(heads, kv_heads, dim, scale, chunk=None, rot=None):
    """The first kind of attention: the values are the keys, so there is no value size of its own."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = rot
    return m


def attn2(heads, kv_heads, dim, vdim, scale, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def ret(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        m["rot"] = rot
    return m


def moe(experts, identity, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(vocab, width, eps, emb_scale, softcap, layers):
    return {"architecture": "Mokalorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb_scale},
            "logit_softcap": softcap, "layers": layers}


# every mixer; grouped kv heads; a chunk that is a multiple of nothing; part of a head rotated; a value size above and below the
# key size; identity experts; a layer without a feed-forward
MOK_A = model(131, 64, 1e-5, 4.0, 10.0, [
    layer("attention", attn(4, 2, 16, 0.3, chunk=11, rot={"base": 100.0, "dims": 8}), moe(5, 2, 3, 40, 0.8)),
    layer("retention", ret(2, 16, 24, [0.9, 0.97], rot={"base": 50.0, "dims": 16}), moe(3, 1, 2, 24, 2.0)),
    layer("attention_2", attn2(3, 1, 24, 20, 0.25, q_temp=(0.7, 5))),
    layer("retention", ret(3, 24, 8, [0.5, 1.0, 0.999], rot={"base": 1e4, "dims": 6}), moe(5, 2, 3, 40, 0.8)),
    layer("attention", attn(4, 2, 16, 0.3, chunk=11, rot={"base": 100.0, "dims": 8}))])

# sizes that are multiples of nothing; one kv head per head; every value rotated; a chunk of one position and one of a page;
# a temperature that changes at every position; no identity experts and one choice; one real expert among identity experts
MOK_B = model(97, 50, 3e-4, 0.5, 4.0, [
    layer("attention_2", attn2(3, 3, 10, 14, 0.4, q_temp=(1.5, 1)), moe(4, 0, 1, 30, 0.5)),
    layer("attention", attn(3, 3, 10, 0.4, chunk=1, rot={"base": 30.0, "dims": 10}), moe(1, 3, 2, 18, 5.0)),
    layer("retention", ret(3, 12, 10, [0.8, 0.8, 0.8], rot={"base": 10.0, "dims": 4})),
    layer("attention", attn(2, 1, 12, 0.25, chunk=8, rot={"base": 1e6, "dims": 2}), moe(4, 0, 1, 30, 0.5)),
    layer("attention_2", attn2(2, 2, 12, 12, 0.3, q_temp=(-0.2, 16)))])

# head sizes the tensor-core attention kernels take (64 and 128 values), a chunk of several pages and one that no page edge meets
MOK_C = model(120, 128, 1e-6, 8.0, 12.0, [
    layer("attention", attn(8, 2, 64, 0.125, chunk=32, rot={"base": 1000.0, "dims": 16}), moe(8, 1, 2, 64, 1.0)),
    layer("attention_2", attn2(4, 1, 128, 128, 0.09, q_temp=(0.3, 20)), moe(8, 1, 2, 64, 1.0)),
    layer("retention", ret(2, 64, 64, [0.99, 0.9], rot={"base": 1e5, "dims": 64}), moe(6, 2, 4, 32, 1.5)),
    layer("attention", attn(2, 2, 128, 0.09, chunk=70, rot={"base": 500.0, "dims": 128}))])

# no logit cap; no rotation anywhere; no query temperature; a chunk longer than every request; every expert chosen; no decay at
# all and a state that keeps little (one that keeps nothing is ill-conditioned under the head norm wherever q . k nearly cancels:
# the retention test covers it alone); feed-forwards that differ from layer to layer
MOK_D = model(80, 40, 1e-5, 1.0, None, [
    layer("retention", ret(2, 20, 20, [1.0, 0.25]), moe(2, 1, 3, 16, 0.3)),
    layer("attention", attn(2, 2, 20, 0.2, chunk=500), moe(3, 0, 2, 44, 3.0)),
    layer("attention_2", attn2(5, 5, 8, 8, 0.35), moe(0, 2, 1, 16, 1.0)),
    layer("attention", attn(1, 1, 40, 0.15, chunk=3))])

ALL = {"A": MOK_A, "B": MOK_B, "C": MOK_C, "D": MOK_D}
