"""Small configurations of the Tifapel decoder for tests.  They differ from one another in every size and
option: head counts and key/value groups, key and value sizes that differ, windows shorter and longer than a
cache page, kept first tokens within and beyond a page, a shared cache entry read under another mask, partial
and full rotation, router groups with one or several kept, one expert per group, a layer without a
feed-forward, a layer without a mask."""


def _moe(experts, top, ff, scale, groups=None):
    r = dict(experts=experts, top=top, scale=scale)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    return dict(kind="moe", expert=dict(ff=ff), router=r)


def _attention(heads, kv_heads, dim, vdim, scale, mask=None, kv_from=None, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if mask:
        m["mask"] = dict(size=mask[0], keep_first=mask[1])
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m, mlp=mlp)


def _retention(heads, dim, vdim, decay, rot, mlp=None):
    return dict(type="retention", mlp=mlp,
                mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay, rot=dict(dims=rot[0], base=rot[1])))


def _lightning(heads, dim, vdim, decay, mlp=None):
    return dict(type="lightning", mlp=mlp, mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay))


# Two key/value groups, values narrower than keys, a window shorter than a page, a reader of layer 0's entry
# with a wider window and fewer kept tokens, partial rotation, groups of which two are kept.
TF_A = dict(
    architecture="Tifapel", vocab=211, width=96, norm=dict(eps=1e-5),
    layers=[
        _attention(4, 2, 32, 16, 0.2, mask=(20, 3), mlp=_moe(8, 3, 40, 2.0, groups=(4, 2))),
        _lightning(3, 16, 24, [0.5, 0.9, 0.99], mlp=_moe(8, 3, 40, 2.0, groups=(4, 2))),
        _retention(2, 32, 40, [0.8, 0.995], rot=(16, 10000.0), mlp=None),
        _attention(4, 2, 32, 16, 0.3, mask=(33, 1), kv_from=0, mlp=_moe(6, 1, 24, 1.0)),
    ])
# Three key/value groups, values wider than keys, windows around and beyond a page, kept tokens beyond a page,
# an attention layer without a mask, one expert per group, full rotation on an odd width.
TF_B = dict(
    architecture="Tifapel", vocab=300, width=100, norm=dict(eps=1e-6),
    layers=[
        _retention(3, 20, 12, [0.3, 0.97, 1.0], rot=(20, 500000.0), mlp=_moe(6, 2, 36, 0.7, groups=(6, 3))),
        _attention(6, 3, 16, 48, 0.25, mask=(64, 70), mlp=_moe(4, 4, 20, 1.3)),
        _attention(3, 3, 48, 48, 0.15, mask=None, mlp=None),
        _attention(6, 3, 16, 48, 0.25, mask=(130, 0), kv_from=1, mlp=_moe(6, 2, 36, 0.7, groups=(3, 1))),
        _lightning(2, 40, 20, [0.9, 0.999], mlp=_moe(10, 2, 16, 2.5, groups=(5, 2))),
    ])
# The sizes the tiled kernels like (multiples of 64 and 128), one kv head, everything else plain.
TF_C = dict(
    architecture="Tifapel", vocab=512, width=256, norm=dict(eps=1e-6),
    layers=[
        _lightning(4, 64, 128, [0.7, 0.9, 0.99, 0.999], mlp=_moe(8, 2, 128, 1.0, groups=(2, 1))),
        _attention(4, 1, 128, 128, 0.09, mask=(100, 2), mlp=_moe(8, 2, 128, 1.0, groups=(2, 1))),
        _retention(2, 128, 64, [0.95, 0.999], rot=(128, 1000000.0), mlp=_moe(8, 2, 128, 1.0, groups=(2, 1))),
    ])
# Head sizes between the tiled kernels' (96: the decode kernel takes it, prompts go to the general kernel; 48 with
# a rotation over 32 dims), as many key/value heads as heads, 20 experts in 5 blocks, a layer that keeps every block.
TF_D = dict(
    architecture="Tifapel", vocab=1000, width=192, norm=dict(eps=1e-6),
    layers=[
        _retention(4, 48, 96, [0.5, 0.9, 0.99, 0.9995], rot=(32, 10000.0), mlp=_moe(20, 3, 72, 1.2, groups=(5, 2))),
        _attention(6, 2, 96, 96, 0.1, mask=(50, 5), mlp=_moe(20, 3, 72, 1.2, groups=(5, 2))),
        _lightning(2, 64, 64, [0.97, 0.999], mlp=_moe(8, 1, 40, 1.0, groups=(4, 4))),
        _attention(6, 2, 96, 96, 0.1, mask=(200, 0), kv_from=1, mlp=None),
        _attention(8, 8, 32, 32, 0.18, mask=(30, 2), mlp=_moe(20, 3, 72, 1.2, groups=(5, 2))),
    ])
ALL = {"A": TF_A, "B": TF_B, "C": TF_C, "D": TF_D}


def make_folder(tmp_path, name: str, dtype: str, seed: int = 4321):
    from pathlib import Path

    from llmoxide_b200.config import read_config
    from llmoxide_b200.weights import write_model_folder

    cfg = dict(ALL[name], torch_dtype=dtype)
    folder = Path(tmp_path) / f"tifapel_{name}_{dtype}"
    if not (folder / "model.safetensors").exists():
        write_model_folder(folder, read_config(cfg), seed, dtype)
    return folder
