"""Measurement (TEST INFRASTRUCTURE, needs a GPU with Triton): which fp32
arithmetic does the GPU compiler emit for the reference's distance predicate

    sqrt(dx*dx + dy*dy + dz*dz) <= radius
    (sparse_engines/strided_grid_radius_triton_kernel.py:25-31,127)?

A Triton kernel written here evaluates that expression on 1,048,576
(query, point) pairs whose distance lies within 3 ulp of the radius, and the
per-query neighbour counts are compared with the library's three predicate
variants (one subprocess each, PCX_RADIUS_PREDICATE=0|1|2).  Result measured on
a B200 with Triton 3.6: the FMA-contracted variants (1, 2) agree with Triton on
every query; the one-rounding-per-operation variant (0) differs on 214 of 4096
queries.  The library therefore defaults to variant 1.

    python oracle/predicate_probe.py
"""
import os, sys, subprocess, json
import numpy as np
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

def make_inputs():
    rng = np.random.default_rng(0)
    Q, per = 4096, 256
    R = 0.05
    q = (rng.random((Q, 3)) * 50).astype(np.float32)        # far apart: no cross pairs
    d = rng.standard_normal((Q, per, 3)); d /= np.linalg.norm(d, axis=-1, keepdims=True)
    scale = R * (1 + rng.integers(-3, 4, (Q, per, 1)) * 2.0 ** -24)
    p = (q[:, None, :].astype(np.float64) + d * scale).astype(np.float32).reshape(-1, 3)
    return q, p, R

if len(sys.argv) > 1 and sys.argv[1] == "lib":
    import torch
    from pointelligence_b200.internals.neighbors import radius_search_sorted_grid8
    q, p, R = make_inputs()
    nb, cnt = radius_search_sorted_grid8(torch.from_numpy(p).cuda(), torch.from_numpy(q).cuda(), R)
    np.save(sys.argv[2], cnt.cpu().numpy())
    sys.exit(0)

import torch, triton, triton.language as tl

@triton.jit
def count_kernel(q_ptr, p_ptr, out_ptr, radius, per: tl.constexpr):
    qi = tl.program_id(0)
    lane = tl.arange(0, per)
    qx = tl.load(q_ptr + qi * 3 + 0); qy = tl.load(q_ptr + qi * 3 + 1); qz = tl.load(q_ptr + qi * 3 + 2)
    base = (qi * per + lane) * 3
    px = tl.load(p_ptr + base + 0); py = tl.load(p_ptr + base + 1); pz = tl.load(p_ptr + base + 2)
    dx = qx - px; dy = qy - py; dz = qz - pz
    dist = tl.sqrt(dx * dx + dy * dy + dz * dz)
    tl.store(out_ptr + qi, tl.sum((dist <= radius).to(tl.int32), axis=0))

q, p, R = make_inputs()
qt, pt = torch.from_numpy(q).cuda(), torch.from_numpy(p).cuda()
out = torch.zeros(len(q), dtype=torch.int32, device="cuda")
count_kernel[(len(q),)](qt, pt, out, float(R), per=256)
tri = out.cpu().numpy().astype(np.int64)
res = {"triton_total": int(tri.sum())}
# IEEE on CPU for orientation
d = (q[:, None, :] - p.reshape(len(q), 256, 3)).astype(np.float32)
s = ((d[..., 0] * d[..., 0]).astype(np.float32) + (d[..., 1] * d[..., 1]).astype(np.float32)).astype(np.float32)
s = (s + (d[..., 2] * d[..., 2]).astype(np.float32)).astype(np.float32)
ieee = (np.sqrt(s).astype(np.float32) <= np.float32(R)).sum(1)
res["ieee_cpu_total"] = int(ieee.sum()); res["queries_differ_triton_vs_ieee"] = int((ieee != tri).sum())
for v in (0, 1, 2):
    f = f"/tmp/cnt{v}.npy"
    env = dict(os.environ, PCX_RADIUS_PREDICATE=str(v))
    subprocess.run([sys.executable, os.path.abspath(__file__), "lib", f], env=env, check=True)
    c = np.load(f)
    res[f"variant{v}_total"] = int(c.sum()); res[f"variant{v}_queries_differ_vs_triton"] = int((c != tri).sum())
print(json.dumps(res))
