"""Dataset loader for static scenes: the metadata logic of the reference's ``load_nerf`` (src/nerf_loader.cu:197-757) and
the pixel conversion of ``convert_rgba32`` (:56-82), for 8-bit images (PNG / JPG through Pillow) of one common resolution.

Returns host arrays in the layout ``Testbed.load_training_data`` takes: RGBA8 pixels (R in the low byte), 3x4 camera-to-world
matrices in the reference's internal convention (``NerfDataset::nerf_matrix_to_ngp``, nerf_loader.h:112-133), focal lengths in
pixels and principal points as fractions of the image.  Not covered (the loader raises instead of guessing): EXR / HDR
images, per-pixel ray files, depth images, lens distortion and rolling shutter, the ``sharpness`` frame filter, the
multi-frame sequences of dynamic scenes.
"""
import json
import math
import os

import numpy as np

NERF_SCALE = 0.33  # nerf_loader.h:31


_F32 = np.float32
_PI_F32 = np.float32(3.14159265358979323846)  # PI() is a float (random_val.cuh:30)


def fov_to_focal_length(resolution, degrees):
    """common_device.cuh:452-454, in single precision like the reference (the tangent is the correctly rounded one, which is what
    the C library's tanf returns)."""
    x = _F32(_F32(_F32(0.5) * _F32(degrees)) * _PI_F32) / _F32(180.0)
    return float(_F32(_F32(0.5) * _F32(resolution)) / _F32(math.tan(float(x))))


def radians_to_degrees(angle):
    """(float)json["camera_angle_x"] * 180 / PI() (nerf_loader.cu:657)"""
    return float(_F32(_F32(angle) * _F32(180.0)) / _PI_F32)


def nerf_matrix_to_ngp(m, scale, offset, from_na=False, from_mitsuba=False):
    """NerfDataset::nerf_matrix_to_ngp (nerf_loader.h:112-133); m is 3x4 (row, column)."""
    r = np.array(m, dtype=np.float32)[:3, :4].copy()
    r[:, 1] *= -1
    r[:, 2] *= -1
    r[:, 3] = r[:, 3] * np.float32(scale) + np.asarray(offset, np.float32)
    if from_na:
        r[:, 1] *= -1
        r[:, 2] *= -1
    elif from_mitsuba:
        r[:, 0] *= -1
        r[:, 2] *= -1
    else:  # cycle axes xyz <- yzx
        r = r[[1, 2, 0], :]
    return r


def ngp_matrix_to_nerf(m, scale, offset, from_na=False, from_mitsuba=False):
    """NerfDataset::ngp_matrix_to_nerf (nerf_loader.h:135-157)."""
    r = np.array(m, dtype=np.float32)[:3, :4].copy()
    if from_na:
        r[:, 1] *= -1
        r[:, 2] *= -1
    elif from_mitsuba:
        r[:, 0] *= -1
        r[:, 2] *= -1
    else:  # cycle axes xyz -> yzx
        r = r[[2, 0, 1], :]
    r[:, 1] *= -1
    r[:, 2] *= -1
    r[:, 3] = (r[:, 3] - np.asarray(offset, np.float32)) / np.float32(scale)
    return r


def _srgb_to_linear(s):
    s = np.asarray(s, np.float32)
    return np.where(s <= 0.04045, s / 12.92, np.power((s + 0.055) / 1.055, 2.4)).astype(np.float32)


def _read_rgba8(path):
    from PIL import Image
    with Image.open(path) as im:
        return np.asarray(im.convert("RGBA"), dtype=np.uint8).copy()  # like stbi_load(..., 4)


def convert_rgba32(rgba, white_transparent=False, black_transparent=False, mask_color=0):
    """convert_rgba32 (src/nerf_loader.cu:56-82) on a [h][w][4] uint8 array; returns [h][w] uint32 (R in the low byte)."""
    px = np.ascontiguousarray(rgba, dtype=np.uint8).copy()
    rgb = px[..., :3]
    if white_transparent:
        px[..., 3][np.all(rgb == 255, axis=-1)] = 0
    if black_transparent:
        px[..., 3][np.all(rgb == 0, axis=-1)] = 0
    packed = px.view(np.uint32)[..., 0]
    if mask_color:
        packed = np.where(packed == np.uint32(mask_color), np.uint32(0x00FF00FF), packed)
    return np.ascontiguousarray(packed)


def _image_path(base, file_path):
    p = os.path.join(base, file_path.replace("\\", "/"))
    if os.path.splitext(p)[1] == "":
        for ext in (".png", ".exr"):
            if os.path.exists(p + ext):
                return p + ext
        raise FileNotFoundError("Could not find image file: " + p)
    return p


def list_frame_jsons(data_path):
    """The per-frame transforms files of a data path (Testbed::load_nerf, src/testbed_nerf.cu:2957-2989): a directory gives every
    *.json in it whose name does not contain "downsample", sorted by base name, one file per frame of a dynamic sequence; a
    single .json is a one-frame sequence."""
    data_path = os.fspath(data_path)
    if os.path.isdir(data_path):
        names = [n for n in os.listdir(data_path)
                 if n.lower().endswith(".json") and "downsample" not in os.path.splitext(n)[0] and os.path.isfile(os.path.join(data_path, n))]
        names.sort(key=lambda n: os.path.splitext(n)[0])
        if not names:
            raise ValueError("NeRF data path contains no json files.")
        return [os.path.join(data_path, n) for n in names]
    if data_path.lower().endswith(".json"):
        return [data_path]
    raise ValueError("NeRF data path must either be a json file or a directory containing json files.")


def load_nerf_dataset(json_paths):
    """json_paths: one transforms file or a list of them.  Returns a dict with pixels [n][h][w] uint32, xforms [n][12] (3x4
    column major), focal [n][2], principal [n][2], and the dataset's scale / offset / aabb_scale / from_na / from_mitsuba /
    render_aabb / up."""
    if isinstance(json_paths, (str, os.PathLike)):
        json_paths = [json_paths]
    if not json_paths:
        raise ValueError("Cannot load NeRF data from an empty set of paths.")
    res = dict(scale=NERF_SCALE, offset=[0.5, 0.5, 0.5], aabb_scale=1, from_na=False, from_mitsuba=False, render_aabb=None,
               up=[0.0, 1.0, 0.0])  # NerfDataset::up (nerf_loader.h:81)
    pixels, xforms, focal, principal = [], [], [], []
    white = black = False
    for jp in json_paths:
        with open(jp) as f:
            js = json.load(f)
        if not isinstance(js.get("frames"), list):
            continue
        base = os.path.dirname(os.path.abspath(jp))
        frames = js["frames"]
        if "n_frames" in js:
            frames = frames[:min(len(frames), int(js["n_frames"]))]
        if frames and "sharpness" in frames[0]:
            raise NotImplementedError("the sharpness frame filter is not built")
        for key in ("k1", "k2", "p1", "p2", "ftheta_p0"):
            if float(js.get(key, 0.0)) != 0.0:
                raise NotImplementedError("lens distortion is not built")
        if "rolling_shutter" in js:
            raise NotImplementedError("rolling shutter is not built")
        if "normal_mts_args" in js:
            res["from_mitsuba"] = True
        if "from_na" in js:
            res["from_na"] = True
        if res["from_mitsuba"]:
            res["scale"] = 0.66
            res["offset"] = [0.25 * 0.66] * 3
        if "render_aabb" in js:
            res["render_aabb"] = np.asarray(js["render_aabb"], np.float32)
        white = bool(js.get("white_transparent", white))
        black = bool(js.get("black_transparent", black))
        if "scale" in js:
            res["scale"] = float(js["scale"])
        # (the file-level cx / cy are parsed by the reference but never reach an image's metadata, nerf_loader.cu:432-438 and
        # :705: the principal point stays at the centre unless a frame carries its own cx / cy or an intrinsic matrix)
        pp = [0.5, 0.5]
        if "aabb_scale" in js:
            res["aabb_scale"] = int(js["aabb_scale"])
        if "offset" in js:
            o = js["offset"]
            res["offset"] = [float(v) for v in o] if isinstance(o, list) else [float(o)] * 3
        if "aabb" in js:  # isotropic fit of the given box into the unit cube, centre at 0.5
            a = np.asarray(js["aabb"], np.float32)
            length = max(1e-6, float(np.abs(a[1] - a[0]).max()))
            res["scale"] = 1.0 / length
            res["offset"] = [float((a[1][e] + a[0][e]) * 0.5 * -res["scale"] + 0.5) for e in range(3)]
        if "up" in js:  # axes permuted like the matrices
            res["up"] = [float(js["up"][1]), float(js["up"][2]), float(js["up"][0])]
        for fr in frames:
            if "transform_matrix_end" in fr and fr["transform_matrix_end"] != fr.get("transform_matrix_start", fr.get("transform_matrix")):
                raise NotImplementedError("moving cameras (transform_matrix_end) are not built")
            path = _image_path(base, fr["file_path"])
            if path.lower().endswith(".exr"):
                raise NotImplementedError("EXR images are not built")
            img = _read_rgba8(path)
            h, w = img.shape[:2]
            alpha_path = os.path.join(base, fr["file_path"] + ".alpha" + os.path.splitext(path)[1])
            if os.path.exists(alpha_path):
                al = _read_rgba8(alpha_path)
                if al.shape[:2] != (h, w):
                    raise ValueError("Alpha image has wrong resolution: " + alpha_path)
                img[..., 3] = (255.0 * _srgb_to_linear(al[..., 0].astype(np.float32) * np.float32(1.0 / 255.0))).astype(np.uint8)
            mask_color = 0
            mask_path = os.path.join(os.path.dirname(path), "dynamic_mask_" + os.path.splitext(os.path.basename(path))[0] + ".png")
            if os.path.exists(mask_path):
                mk = _read_rgba8(mask_path)
                if mk.shape[:2] != (h, w):
                    raise ValueError("Mask image has wrong resolution: " + mask_path)
                mask_color = 0x00FF00FF
                img.view(np.uint32)[..., 0][mk[..., 0] != 0] = mask_color
            pixels.append(convert_rgba32(img, white, black, mask_color))

            def read_focal_length(resolution, axis):
                if axis + "_fov" in fr:
                    return fov_to_focal_length(resolution, float(fr[axis + "_fov"]))
                if "fl_" + axis in js:
                    return float(js["fl_" + axis])
                if "camera_angle_" + axis in js:
                    return fov_to_focal_length(resolution, radians_to_degrees(js["camera_angle_" + axis]))
                if "fl_" + axis in fr:
                    return float(fr["fl_" + axis])
                if "camera_angle_" + axis in fr:
                    return fov_to_focal_length(resolution, radians_to_degrees(fr["camera_angle_" + axis]))
                return 0.0
            x_fl, y_fl = read_focal_length(w, "x"), read_focal_length(h, "y")
            p = list(pp)
            if x_fl != 0:
                fl = [x_fl, y_fl if y_fl != 0 else x_fl]
            elif y_fl != 0:
                fl = [y_fl, y_fl]
            elif "intrinsic_matrix" in fr:
                k = fr["intrinsic_matrix"]
                fl = [float(k[0][0]), float(k[1][1])]
                p = [float(k[0][2]) / float(js["w"]), float(k[1][2]) / float(js["h"])]
            else:
                raise ValueError("Couldn't read fov.")
            if "cx" in fr:
                p[0] = float(fr["cx"]) / float(fr["w"])
            if "cy" in fr:
                p[1] = float(fr["cy"]) / float(fr["h"])
            focal.append(fl)
            principal.append(p)
            m = fr["transform_matrix_start"] if "transform_matrix_start" in fr else fr["transform_matrix"]
            ngp = nerf_matrix_to_ngp(np.asarray(m, np.float32), res["scale"], res["offset"], res["from_na"], res["from_mitsuba"])
            xforms.append(ngp.T.reshape(-1))  # column major
    if not pixels:
        raise ValueError("No training images were found for NeRF training!")
    shapes = {p.shape for p in pixels}
    if len(shapes) != 1:
        raise NotImplementedError(f"images of different resolutions are not built: {sorted(shapes)}")
    res.update(pixels=np.stack(pixels), xforms=np.asarray(xforms, np.float32), focal=np.asarray(focal, np.float32),
               principal=np.asarray(principal, np.float32), n_images=len(pixels))
    return res
