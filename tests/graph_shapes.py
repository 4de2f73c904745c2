"""Small multi-branch graphs shared by the CPU (dry-run: dependency structure) and GPU (numerics) tests.  They restate
the graph shapes of the reference's test-mode suite (tests/runtime_python/test_mode/test_{fork_point,join_point,
diamond_fork_join,residual_stripping,grid_dim_sweep,case2_case3_negative}_testmode.py): a producer with two
consumers, a consumer with two producers, both at once, a residual shortcut beside a longer path, and the two role
combinations the reference's event model has to refuse (a task there carries one trigger and one dependent event;
here a layer triggers one event and waits for up to three, so those graphs are ordinary)."""
import torch


def build(pk, kind, B, H, dev):
    """Registers graph `kind` on `pk`; returns ({name: host input}, {name: device output}, reference function)."""
    g = torch.Generator().manual_seed(hash(kind) % 1000 + B + H)
    bf = torch.bfloat16
    rnd = lambda *s, scale=1.0, shift=0.0: (shift + scale * torch.randn(*s, generator=g)).to(bf)
    t = {}

    def inp(name, *shape, **kw):
        t[name] = rnd(*shape, **kw)
        return pk.attach_input(t[name].to(dev) if dev != "meta" else torch.empty(*shape, dtype=bf, device="meta"), name)

    outs = {}

    def out(name, *shape):
        outs[name] = torch.zeros(*shape, dtype=bf, device=dev) if dev != "meta" else torch.empty(*shape, dtype=bf, device="meta")
        return pk.attach_input(outs[name], name)

    norm = lambda x, w, o: pk.rmsnorm_layer(input=x, weight=w, output=o, grid_dim=(B, 1, 1), block_dim=(128, 1, 1))
    lin = lambda x, w, o: pk.linear_layer(input=x, weight=w, output=o, grid_dim=(H // 64, 1, 1), block_dim=(128, 1, 1))
    linres = lambda x, w, r, o: pk.linear_with_residual_layer(input=x, weight=w, residual=r, output=o,
                                                              grid_dim=(H // 64, 1, 1), block_dim=(128, 1, 1))
    x = inp("x", B, H)
    from oracle import mpk_ops as ops
    if kind == "fork":
        wa, wb, wc = inp("wa", H, shift=1, scale=.1), inp("wb", H, shift=1, scale=.1), inp("wc", H, shift=1, scale=.1)
        xa, xb, xc = out("xa", B, H), out("xb", B, H), out("xc", B, H)
        norm(x, wa, xa); norm(xa, wb, xb); norm(xa, wc, xc)

        def ref():
            a = ops.rmsnorm(t["x"], t["wa"], 1e-6)
            return {"xa": a, "xb": ops.rmsnorm(a, t["wb"], 1e-6), "xc": ops.rmsnorm(a, t["wc"], 1e-6)}
    elif kind == "join":
        y = inp("y", B, H)
        wa, wb, wc = inp("wa", H, shift=1, scale=.1), inp("wb", H, shift=1, scale=.1), inp("wc", H, H, scale=.02)
        xa, xb, xc = out("xa", B, H), out("xb", B, H), out("xc", B, H)
        norm(x, wa, xa); norm(y, wb, xb); linres(xa, wc, xb, xc)

        def ref():
            a, b = ops.rmsnorm(t["x"], t["wa"], 1e-6), ops.rmsnorm(t["y"], t["wb"], 1e-6)
            return {"xc": ops.linear(a, t["wc"], b)}
    elif kind == "diamond":
        wa = inp("wa", H, shift=1, scale=.1)
        wb, wc, wd = inp("wb", H, H, scale=.02), inp("wc", H, H, scale=.02), inp("wd", H, H, scale=.02)
        xa, xb, xc, xd = out("xa", B, H), out("xb", B, H), out("xc", B, H), out("xd", B, H)
        norm(x, wa, xa); lin(xa, wb, xb); lin(xa, wc, xc); linres(xb, wd, xc, xd)

        def ref():
            a = ops.rmsnorm(t["x"], t["wa"], 1e-6)
            b, c = ops.linear(a, t["wb"]), ops.linear(a, t["wc"])
            return {"xd": ops.linear(b, t["wd"], c)}
    elif kind == "residual_shortcut":
        wa, wb, wc = inp("wa", H, shift=1, scale=.1), inp("wb", H, shift=1, scale=.1), inp("wc", H, H, scale=.02)
        xa, xb, xc = out("xa", B, H), out("xb", B, H), out("xc", B, H)
        norm(x, wa, xa); norm(xa, wb, xb); linres(xb, wc, xa, xc)

        def ref():
            a = ops.rmsnorm(t["x"], t["wa"], 1e-6)
            return {"xc": ops.linear(ops.rmsnorm(a, t["wb"], 1e-6), t["wc"], a)}
    elif kind == "join_and_fork_consumer":       # the reference's "case 2"
        y = inp("y", B, H)
        wa, we, wc = inp("wa", H, shift=1, scale=.1), inp("we", H, shift=1, scale=.1), inp("wc", H, shift=1, scale=.1)
        wb = inp("wb", H, H, scale=.02)
        xa, xe, xb, xc = out("xa", B, H), out("xe", B, H), out("xb", B, H), out("xc", B, H)
        norm(x, wa, xa); norm(y, we, xe)
        linres(xa, wb, xe, xb)                   # waits for A (which also feeds C: a fork) and for E (a join)
        norm(xa, wc, xc)

        def ref():
            a, e = ops.rmsnorm(t["x"], t["wa"], 1e-6), ops.rmsnorm(t["y"], t["we"], 1e-6)
            return {"xb": ops.linear(a, t["wb"], e), "xc": ops.rmsnorm(a, t["wc"], 1e-6)}
    elif kind == "fork_and_join_producer":       # the reference's "case 3"
        y = inp("y", B, H)
        wa, we, wc = inp("wa", H, shift=1, scale=.1), inp("we", H, shift=1, scale=.1), inp("wc", H, shift=1, scale=.1)
        wd = inp("wd", H, H, scale=.02)
        xa, xe, xc, xd = out("xa", B, H), out("xe", B, H), out("xc", B, H), out("xd", B, H)
        norm(x, wa, xa); norm(y, we, xe)
        norm(xa, wc, xc)                         # A feeds C and D (a fork) ...
        linres(xa, wd, xe, xd)                   # ... and, with E, the join D

        def ref():
            a, e = ops.rmsnorm(t["x"], t["wa"], 1e-6), ops.rmsnorm(t["y"], t["we"], 1e-6)
            return {"xc": ops.rmsnorm(a, t["wc"], 1e-6), "xd": ops.linear(a, t["wd"], e)}
    else:
        raise KeyError(kind)
    return t, outs, ref


KINDS = ("fork", "join", "diamond", "residual_shortcut", "join_and_fork_consumer", "fork_and_join_producer")
