"""Seeded synthetic scenes in the reference's data convention (RGBA8 images with the mask in alpha, 3x4 camera-to-world
matrices already in the unit-cube frame the testbed trains in, pinhole intrinsics in pixels).

They stand in for the DTU-style captures the reference is run on: an analytic sphere (radius 0.3, centred in the unit
cube) with a 3-octave value-noise albedo, Lambert + ambient shading, cameras on a Fibonacci sphere looking at the
centre.  Everything is generated with torch so it can be made directly on the GPU for benchmarks or on the CPU for the
oracle tests; it is input preparation, not part of the timed path."""
import math

import numpy as np
import torch


def fibonacci_cameras(n_views, radius=2.5, center=(0.5, 0.5, 0.5)):
    """[n][12] column-major 3x4 camera-to-world matrices: columns right, down, forward, origin."""
    out = np.zeros((n_views, 12), np.float32)
    golden = math.pi * (3.0 - math.sqrt(5.0))
    c = np.asarray(center, np.float64)
    for i in range(n_views):
        z = 1.0 - 2.0 * (i + 0.5) / n_views
        r = math.sqrt(max(0.0, 1.0 - z * z))
        th = golden * i
        n = np.array([r * math.cos(th), r * math.sin(th), z])
        origin = c + radius * n
        fwd = -n
        up = np.array([0.0, 0.0, 1.0]) if abs(n[2]) < 0.99 else np.array([0.0, 1.0, 0.0])
        right = np.cross(fwd, up)
        right /= np.linalg.norm(right)
        down = np.cross(fwd, right)
        out[i, 0:3], out[i, 3:6], out[i, 6:9], out[i, 9:12] = right, down, fwd, origin
    return out


def _value_noise(p, seed, octaves=3, base_freq=4.0):
    """3-channel value noise in [0,1]: trilinear interpolation of a seeded random lattice, summed over octaves."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    out = torch.zeros(p.shape[0], 3, device=p.device)
    amp_sum = 0.0
    for o in range(octaves):
        freq, amp = base_freq * (2 ** o), 0.5 ** o
        res = int(freq) + 2
        table = torch.rand((res, res, res, 3), generator=g).to(p.device)
        q = p * freq
        q0 = torch.floor(q)
        f = q - q0
        i0 = q0.long().clamp(0, res - 2)
        acc = 0
        for k in range(8):
            b = [(k >> e) & 1 for e in range(3)]
            w = 1.0
            for e in range(3):
                w = w * (f[:, e] if b[e] else 1.0 - f[:, e])
            acc = acc + w[:, None] * table[i0[:, 0] + b[0], i0[:, 1] + b[1], i0[:, 2] + b[2]]
        out += amp * acc
        amp_sum += amp
    return out / amp_sum


def _linear_to_srgb(x):
    return torch.where(x < 0.0031308, 12.92 * x, 1.055 * x.clamp_min(1e-8) ** (1 / 2.4) - 0.055)


def sequence_poses(n_frames, seed=0, max_rot_deg=5.0, max_shift=0.02, bulge=0.03, bulge_period=25.0, radius=0.3):
    """Per-frame pose of the moving sphere of the dynamic stand-in sequence: a seeded random walk of rigid motions (each step a
    rotation of at most `max_rot_deg` about a random axis and a translation of at most `max_shift`) and a sinusoidal radial
    bulge.  Returns [(rotation [3][3], translation [3], radius)] with the identity first."""
    rng = np.random.default_rng(seed)
    R, t, out = np.eye(3), np.zeros(3), []
    for f in range(n_frames):
        out.append((R.astype(np.float32), t.astype(np.float32), float(radius + bulge * math.sin(2.0 * math.pi * f / bulge_period))))
        axis = rng.normal(size=3)
        axis /= np.linalg.norm(axis)
        ang = math.radians(max_rot_deg) * rng.uniform(0.3, 1.0)
        K = np.array([[0, -axis[2], axis[1]], [axis[2], 0, -axis[0]], [-axis[1], axis[0], 0]])
        step = np.eye(3) + math.sin(ang) * K + (1 - math.cos(ang)) * (K @ K)
        R = step @ R
        shift = rng.normal(size=3)
        t = t + max_shift * rng.uniform(0.3, 1.0) * shift / np.linalg.norm(shift)
    return out


def render_sphere_views(n_views=64, width=512, height=512, fov_deg=40.0, radius=0.3, seed=0, device="cpu", cam_radius=2.5,
                        rotation=None, translation=None):
    """Returns dict(pixels int32 [n][H][W] (RGBA8, R low byte), xforms [n][12], focal [n][2], principal [n][2]).
    `rotation` [3][3] / `translation` [3] move the object rigidly about the cube's centre (its albedo moves with it); the
    cameras and the light stay."""
    xforms = torch.from_numpy(fibonacci_cameras(n_views, cam_radius)).to(device)
    focal_px = 0.5 * width / math.tan(0.5 * math.radians(fov_deg))
    focal = torch.full((n_views, 2), focal_px, dtype=torch.float32, device=device)
    principal = torch.full((n_views, 2), 0.5, dtype=torch.float32, device=device)
    ys, xs = torch.meshgrid(torch.arange(height, device=device), torch.arange(width, device=device), indexing="ij")
    u = ((xs.float() + 0.5) / width).reshape(-1)
    v = ((ys.float() + 0.5) / height).reshape(-1)
    dl = torch.stack([(u - 0.5) * width / focal_px, (v - 0.5) * height / focal_px, torch.ones_like(u)], 1)
    cube_center = torch.tensor([0.5, 0.5, 0.5], device=device)
    Robj = torch.eye(3, device=device) if rotation is None else torch.as_tensor(np.asarray(rotation, np.float32), device=device)
    tobj = torch.zeros(3, device=device) if translation is None else torch.as_tensor(np.asarray(translation, np.float32), device=device)
    center = cube_center + tobj
    light = torch.tensor([0.4, -0.5, 0.77], device=device)
    light = light / light.norm()
    pixels = torch.zeros((n_views, height, width), dtype=torch.int32, device=device)
    for i in range(n_views):
        X = xforms[i]
        R = torch.stack([X[0:3], X[3:6], X[6:9]], 1)  # columns
        o = X[9:12]
        d = dl @ R.T
        d = d / d.norm(dim=1, keepdim=True)
        oc = o - center
        b = (d * oc).sum(1)
        disc = b * b - (oc @ oc - radius * radius)
        hit = disc > 0
        t = -b - torch.sqrt(disc.clamp_min(0))
        p = o + t[:, None] * d
        nrm = (p - center) / radius
        q = (p - center) @ Robj + cube_center  # the point in the object's own frame: R^T (p - c - t) + c
        albedo = 0.15 + 0.8 * _value_noise(q.clamp(0, 1), seed)
        shade = 0.3 + 0.7 * (nrm @ light).clamp_min(0)
        col = _linear_to_srgb((albedo * shade[:, None]).clamp(0, 1))
        rgb8 = (col * 255.0 + 0.5).clamp(0, 255).to(torch.int64)
        rgb8 = torch.where(hit[:, None], rgb8, torch.zeros_like(rgb8))
        a8 = torch.where(hit, 255, 0).to(torch.int64)
        packed = rgb8[:, 0] | (rgb8[:, 1] << 8) | (rgb8[:, 2] << 16) | (a8 << 24)
        packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed)  # keep the bit pattern in int32
        pixels[i] = packed.to(torch.int32).reshape(height, width)
    return dict(pixels=pixels, xforms=xforms, focal=focal, principal=principal, width=width, height=height)


def csg_sdf(p, center=(0.5, 0.5, 0.5)):
    """Signed distance of the union of a torus (R 0.25, r 0.08, axis z) and a rounded box (half-extent 0.15, corner radius
    0.02), both centred in the unit cube; p is [n][3] (torch)."""
    q = p - torch.tensor(center, device=p.device, dtype=p.dtype)
    ring = torch.sqrt(q[:, 0] ** 2 + q[:, 1] ** 2) - 0.25
    torus = torch.sqrt(ring ** 2 + q[:, 2] ** 2) - 0.08
    d = q.abs() - (0.15 - 0.02)
    box = d.clamp_min(0).norm(dim=1) + d.max(dim=1).values.clamp_max(0) - 0.02
    return torch.minimum(torus, box)


def cap_cameras(n_views, radius=2.5, cap_deg=60.0, center=(0.5, 0.5, 0.5)):
    """[n][12] camera-to-world matrices on a spherical cap of half-angle cap_deg around +z, looking at the centre."""
    out = np.zeros((n_views, 12), np.float32)
    golden = math.pi * (3.0 - math.sqrt(5.0))
    c = np.asarray(center, np.float64)
    zmin = math.cos(math.radians(cap_deg))
    for i in range(n_views):
        z = 1.0 - (1.0 - zmin) * (i + 0.5) / n_views
        r = math.sqrt(max(0.0, 1.0 - z * z))
        th = golden * i
        n = np.array([r * math.cos(th), r * math.sin(th), z])
        fwd = -n
        up = np.array([0.0, 0.0, 1.0]) if abs(n[2]) < 0.99 else np.array([0.0, 1.0, 0.0])
        right = np.cross(fwd, up)
        right /= np.linalg.norm(right)
        down = np.cross(fwd, right)
        out[i, 0:3], out[i, 3:6], out[i, 6:9], out[i, 9:12] = right, down, fwd, c + radius * n
    return out


def render_csg_views(n_views=49, width=1600, height=1200, fov_deg=30.0, seed=0, device="cpu", cam_radius=2.5, chunk=1 << 21):
    """The DTU-shaped stand-in scene: torus + rounded box (csg_sdf) with a checker / value-noise albedo, sphere-traced from
    cameras on a 60-degree cap.  Same dict as render_sphere_views."""
    xforms = torch.from_numpy(cap_cameras(n_views, cam_radius)).to(device)
    focal_px = 0.5 * width / math.tan(0.5 * math.radians(fov_deg))
    focal = torch.full((n_views, 2), focal_px, dtype=torch.float32, device=device)
    principal = torch.full((n_views, 2), 0.5, dtype=torch.float32, device=device)
    ys, xs = torch.meshgrid(torch.arange(height, device=device), torch.arange(width, device=device), indexing="ij")
    u = ((xs.float() + 0.5) / width).reshape(-1)
    v = ((ys.float() + 0.5) / height).reshape(-1)
    dl = torch.stack([(u - 0.5) * width / focal_px, (v - 0.5) * height / focal_px, torch.ones_like(u)], 1)
    light = torch.tensor([0.4, -0.5, 0.77], device=device)
    light = light / light.norm()
    pixels = torch.zeros((n_views, height * width), dtype=torch.int32, device=device)
    eps = 1e-3
    for i in range(n_views):
        X = xforms[i]
        R = torch.stack([X[0:3], X[3:6], X[6:9]], 1)
        o = X[9:12]
        for c0 in range(0, height * width, chunk):
            d = dl[c0:c0 + chunk] @ R.T
            d = d / d.norm(dim=1, keepdim=True)
            t = torch.full((d.shape[0],), cam_radius - 0.75, device=device)
            for _ in range(96):  # sphere tracing
                t = t + csg_sdf(o + t[:, None] * d)
                t = t.clamp_max(cam_radius + 0.75)
            p = o + t[:, None] * d
            hit = csg_sdf(p).abs() < 2e-4
            g = torch.stack([csg_sdf(p + torch.tensor(e, device=device)) - csg_sdf(p - torch.tensor(e, device=device))
                             for e in ((eps, 0, 0), (0, eps, 0), (0, 0, eps))], 1)
            nrm = g / g.norm(dim=1, keepdim=True).clamp_min(1e-12)
            pc = p.clamp(0, 1)
            checker = ((torch.floor(pc[:, 0] * 8) + torch.floor(pc[:, 1] * 8) + torch.floor(pc[:, 2] * 8)) % 2)[:, None]
            albedo = (0.15 + 0.8 * _value_noise(pc, seed)) * (0.6 + 0.4 * checker)
            shade = 0.3 + 0.7 * (nrm @ light).clamp_min(0)
            col = _linear_to_srgb((albedo * shade[:, None]).clamp(0, 1))
            rgb8 = (col * 255.0 + 0.5).clamp(0, 255).to(torch.int64)
            rgb8 = torch.where(hit[:, None], rgb8, torch.zeros_like(rgb8))
            a8 = torch.where(hit, 255, 0).to(torch.int64)
            packed = rgb8[:, 0] | (rgb8[:, 1] << 8) | (rgb8[:, 2] << 16) | (a8 << 24)
            packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed)
            pixels[i, c0:c0 + chunk] = packed.to(torch.int32)
    return dict(pixels=pixels.reshape(n_views, height, width), xforms=xforms, focal=focal, principal=principal, width=width, height=height)


def geometric_init_sdf_weights(seed=7, in_width=48, bias_radius=None):
    """Sphere-like initialisation of the one-hidden-layer SDF net (the role utils/mlp_weights.txt plays in the
    reference, nerf_network.h:774-823): first layer ~ N(0, sqrt(2)/sqrt(64)) on the xyz columns only, last layer
    rows = sqrt(pi)/sqrt(64).  Returns float32 [64*in_width + 16*64], row-major [out][in]."""
    rng = np.random.default_rng(seed)
    W1 = np.zeros((64, in_width), np.float32)
    W1[:, :3] = rng.normal(0.0, math.sqrt(2.0) / math.sqrt(64.0), (64, 3))
    W2 = np.full((16, 64), math.sqrt(math.pi) / math.sqrt(64.0), np.float32)
    return np.concatenate([W1.ravel(), W2.ravel()])


def init_params(grid_n_params, seed=1337, variance=0.3):
    """fp32 master parameters of the whole block: SDF net geometric init, colour net Xavier-uniform, grid U(-1e-4,1e-4)
    (takikawa_encoding.cuh:454 shows the convention), variance 0.3 (nerf_network.h:872)."""
    rng = np.random.default_rng(seed)
    p = np.zeros(12288 + grid_n_params + 4, np.float32)
    p[:4096] = geometric_init_sdf_weights(seed)
    off = 4096
    for (o, i) in ((64, 48), (64, 64), (16, 64)):
        lim = math.sqrt(6.0 / (o + i))
        p[off:off + o * i] = rng.uniform(-lim, lim, o * i)
        off += o * i
    p[12288:12288 + grid_n_params] = rng.uniform(-1e-4, 1e-4, grid_n_params)
    p[12288 + grid_n_params:] = variance
    return p


def write_sequence_dataset(scenes, directory):
    """A dynamic sequence in the reference's layout: one transforms file per frame in one directory (frame_0000.json, ...; the
    loader sorts them by name, src/testbed_nerf.cu:2958-2996), each with its own image folder.  Returns the directory."""
    for f, scene in enumerate(scenes):
        write_transforms_dataset(scene, directory, json_name="frame_%04d.json" % f, image_dir="images_%04d" % f)
    return directory


def write_transforms_dataset(scene, directory, json_name="transforms.json", image_dir="images"):
    """Writes a synthetic scene (the dict of render_sphere_views / render_csg_views) as a dataset in the reference's file format:
    <directory>/transforms.json plus one RGBA PNG per view, with `scale` 1 and `offset` 0 so that the loader's
    nerf_matrix_to_ngp gives back exactly the scene's camera matrices.  Returns the path of the json file."""
    import json
    import os
    from PIL import Image
    from .loader import ngp_matrix_to_nerf
    t = lambda k: scene[k].cpu().numpy() if hasattr(scene[k], "cpu") else np.asarray(scene[k])
    px, xf, fl, pp = t("pixels"), t("xforms"), t("focal"), t("principal")
    n, h, w = px.shape
    os.makedirs(os.path.join(directory, image_dir), exist_ok=True)
    frames = []
    for i in range(n):
        rgba = np.ascontiguousarray(px[i]).view(np.uint8).reshape(h, w, 4)
        Image.fromarray(rgba, "RGBA").save(os.path.join(directory, image_dir, "%04d.png" % i))
        m = np.asarray(xf[i], np.float32).reshape(4, 3).T  # [12] column major -> 3x4
        nerf = ngp_matrix_to_nerf(m, 1.0, [0.0, 0.0, 0.0])
        frames.append({"file_path": "%s/%04d.png" % (image_dir, i), "transform_matrix": np.vstack([nerf, [0, 0, 0, 1]]).astype(float).tolist(),
                       "fl_x": float(fl[i][0]), "fl_y": float(fl[i][1]), "cx": float(pp[i][0] * w), "cy": float(pp[i][1] * h), "w": w, "h": h})
    js = {"scale": 1.0, "offset": [0.0, 0.0, 0.0], "aabb_scale": 1, "w": w, "h": h, "fl_x": float(fl[0][0]), "fl_y": float(fl[0][1]),
          "cx": float(pp[0][0] * w), "cy": float(pp[0][1] * h), "frames": frames}
    path = os.path.join(directory, json_name)
    with open(path, "w") as f:
        json.dump(js, f)
    return path

