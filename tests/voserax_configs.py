"""Small configurations of the Voserax decoder for tests.  They differ from one another in every size and option:
stream counts (none, 1, 2, 3, 5), head counts and key/value groups, key and value sizes that differ or agree, windows
shorter and longer than a cache page or none, 2 to 5 convolution taps or none, partial, full or no rotation with and
without scaled frequencies, value mixing that starts at a later layer or is absent, dense, routed and absent
feed-forwards in any order, routers with and without identity experts, shared experts and more than one choice."""


def _attention(heads, kv_heads, dim, vdim, scale, window=None, conv=None, rot=None, scaling=None, v_mix=False, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if window:
        m["mask"] = dict(size=window)
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = dict(dims=rot[0], base=rot[1])
        if scaling:
            m["rot"]["scaling"] = dict(factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
    if v_mix:
        m["v_mix"] = True
    return dict(type="attention", mixer=m, mlp=mlp)


def _dense(ff):
    return dict(kind="dense", ff=ff)


def _moe(experts, top, ff, limit, identity=0, shared=None):
    mlp = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top, identity=identity))
    if shared:
        mlp["shared"] = dict(ff=shared[0], limit=shared[1])
    return mlp


# Three streams, two key/value groups, values narrower than keys, a window shorter than a page, 3 taps, partial
# rotation with scaled frequencies, mixing from the second layer on, a dense and two routed feed-forwards.
VX_A = dict(
    architecture="Voserax", vocab=211, width=96, norm=dict(eps=1e-5), residual_mult=0.5, streams=3, max_positions=512,
    layers=[
        _attention(4, 2, 32, 16, 0.2, window=20, conv=3, rot=(16, 10000.0), scaling=(4.0, 64, 8.0, 1.0), mlp=_dense(72)),
        _attention(4, 2, 32, 16, 0.25, window=33, conv=3, rot=(16, 10000.0), v_mix=True,
                   mlp=_moe(6, 2, 40, 1.5, identity=2, shared=(24, 0.8))),
        _attention(2, 1, 48, 32, 0.15, window=7, conv=2, rot=(48, 500.0), scaling=(2.0, 128, 16.0, 2.0), v_mix=False,
                   mlp=None),
        _attention(6, 2, 16, 16, 0.3, window=64, conv=3, v_mix=True, mlp=_moe(5, 1, 24, 3.0, identity=0, shared=None)),
    ])
# One stream with connection weights, three key/value groups, values wider than keys, windows around and beyond a
# page and none at all, 5 taps and none, every layer mixes, top 3 of 4 + 3 identity experts.
VX_B = dict(
    architecture="Voserax", vocab=300, width=100, norm=dict(eps=1e-6), residual_mult=1.0, streams=1, max_positions=400,
    layers=[
        _attention(6, 3, 16, 48, 0.25, window=65, conv=5, rot=(8, 100.0), v_mix=True, mlp=_moe(4, 3, 20, 0.7, identity=3)),
        _attention(3, 3, 24, 48, 0.2, window=None, conv=None, rot=(24, 10000.0), v_mix=True, mlp=_dense(36)),
        _attention(6, 3, 16, 48, 0.25, window=130, conv=4, v_mix=True,
                   mlp=_moe(7, 2, 16, 2.0, identity=1, shared=(40, 2.0))),
    ])
# The sizes the tiled kernels like (64 and 128, keys and values alike), one key/value head, two and five streams.
VX_C = dict(
    architecture="Voserax", vocab=500, width=256, norm=dict(eps=1e-6), residual_mult=0.8, streams=2, max_positions=1024,
    layers=[
        _attention(4, 1, 128, 128, 0.09, window=100, conv=4, rot=(64, 10000.0), scaling=(2.0, 256, 32.0, 1.0), v_mix=True,
                   mlp=_moe(12, 2, 128, 1.25, identity=1, shared=(128, 1.25))),
        _attention(4, 2, 64, 64, 0.12, window=70, conv=4, rot=(64, 10000.0), mlp=_dense(256)),
        _attention(4, 1, 128, 128, 0.09, window=300, conv=2, rot=(128, 1000000.0), v_mix=True,
                   mlp=_moe(12, 2, 128, 1.25, identity=1, shared=(128, 1.25))),
    ])
# No hyper-connections at all (plain residual sums times the factor); a layer without convolution, rotation or
# window, and one whose window is a single token and whose router takes every expert.
VX_D = dict(
    architecture="Voserax", vocab=130, width=64, norm=dict(eps=1e-5), residual_mult=0.9, max_positions=300,
    layers=[
        _attention(2, 2, 32, 32, 0.2, mlp=_dense(48)),
        _attention(2, 1, 32, 8, 0.2, window=1, conv=2, mlp=_moe(3, 3, 16, 1.0)),
    ])
# Five streams, one key/value head, values wider than keys, top 4 of 9 + 4 identity experts, a layer without a
# feed-forward in the middle, a window of five tokens.
VX_E = dict(
    architecture="Voserax", vocab=160, width=72, norm=dict(eps=1e-5), residual_mult=0.7, streams=5, max_positions=300,
    layers=[
        _attention(3, 1, 24, 40, 0.3, window=41, conv=4, rot=(12, 10000.0), scaling=(8.0, 32, 4.0, 1.0), v_mix=True,
                   mlp=_moe(9, 4, 24, 1.0, identity=4, shared=(16, 1.0))),
        _attention(3, 1, 24, 40, 0.3, window=41, conv=4, rot=(12, 10000.0), scaling=(8.0, 32, 4.0, 1.0), v_mix=True,
                   mlp=None),
        _attention(3, 1, 24, 40, 0.3, window=5, conv=4, rot=(12, 10000.0), v_mix=True, mlp=_dense(30)),
    ])
ALL = {"A": VX_A, "B": VX_B, "C": VX_C, "D": VX_D, "E": VX_E}


def make_folder(tmp_path, name: str, dtype: str, seed: int = 977):
    from pathlib import Path

    from llmoxide_b200.config import read_config
    from llmoxide_b200.weights import write_model_folder

    cfg = dict(ALL[name], torch_dtype=dtype)
    folder = Path(tmp_path) / f"voserax_{name}_{dtype}"
    if not (folder / "model.safetensors").exists():
        write_model_folder(folder, read_config(cfg), seed, dtype)
    return folder
