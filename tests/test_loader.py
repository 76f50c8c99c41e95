"""Dataset loader (host logic): the metadata rules of the reference's load_nerf on small generated scenes."""
import json
import math

import numpy as np
import pytest


def write_scene(tmp_path, extra=None, frame_extra=None, n=3, w=8, h=6, ext="png"):
    from PIL import Image
    rng = np.random.default_rng(0)
    frames, images = [], []
    (tmp_path / "images").mkdir(exist_ok=True)
    for i in range(n):
        img = rng.integers(0, 256, (h, w, 4), dtype=np.uint8)
        img[0, 0] = (255, 255, 255, 255)
        img[0, 1] = (0, 0, 0, 255)
        Image.fromarray(img, "RGBA").save(tmp_path / "images" / f"{i:03d}.{ext}")
        images.append(img)
        m = np.eye(4)
        m[:3, :3] = np.linalg.qr(rng.normal(size=(3, 3)))[0]
        m[:3, 3] = rng.normal(size=3)
        fr = {"file_path": f"images/{i:03d}" if i % 2 else f"images/{i:03d}.{ext}", "transform_matrix": m.tolist()}
        fr.update(frame_extra or {})
        frames.append(fr)
    js = {"camera_angle_x": 0.7, "frames": frames}
    js.update(extra or {})
    (tmp_path / "transforms.json").write_text(json.dumps(js))
    return tmp_path / "transforms.json", images, frames


def test_default_conventions(tmp_path):
    from neus2_b200 import loader
    path, images, frames = write_scene(tmp_path)
    ds = loader.load_nerf_dataset(path)
    assert ds["n_images"] == 3 and ds["pixels"].shape == (3, 6, 8) and ds["pixels"].dtype == np.uint32
    np.testing.assert_array_equal(ds["pixels"][1].view(np.uint8).reshape(6, 8, 4), images[1])  # R in the low byte
    f = 0.5 * 8 / math.tan(0.5 * 0.7)
    np.testing.assert_allclose(ds["focal"], f, rtol=1e-6)
    np.testing.assert_array_equal(ds["principal"], 0.5)
    assert ds["scale"] == pytest.approx(0.33) and ds["offset"] == [0.5, 0.5, 0.5] and ds["aabb_scale"] == 1
    # nerf_matrix_to_ngp: columns 1, 2 negated, translation scaled and offset, rows cycled (x <- y, y <- z, z <- x)
    m = np.asarray(frames[0]["transform_matrix"], np.float32)[:3]
    exp = m.copy()
    exp[:, 1:3] *= -1
    exp[:, 3] = exp[:, 3] * np.float32(0.33) + 0.5
    exp = exp[[1, 2, 0]]
    got = ds["xforms"][0].reshape(4, 3).T
    np.testing.assert_allclose(got, exp, rtol=1e-6)
    back = loader.ngp_matrix_to_nerf(got, ds["scale"], ds["offset"])
    np.testing.assert_allclose(back, m, rtol=1e-5, atol=1e-6)


def test_from_na_scale_offset_aabb_and_intrinsics(tmp_path):
    from neus2_b200 import loader
    k = [[700.0, 0, 3.0], [0, 710.0, 2.0], [0, 0, 1]]
    js = {"from_na": True, "w": 8, "h": 6, "aabb_scale": 1, "scale": 0.5, "offset": [0.4, 0.5, 0.6], "cx": 1.0, "cy": 1.0}
    path, _, frames = write_scene(tmp_path, extra=js, frame_extra={"intrinsic_matrix": k})
    raw = json.loads(path.read_text())
    del raw["camera_angle_x"]
    path.write_text(json.dumps(raw))
    ds = loader.load_nerf_dataset([path])
    assert ds["from_na"] and ds["scale"] == 0.5
    np.testing.assert_allclose(ds["focal"], [[700.0, 710.0]] * 3)
    np.testing.assert_allclose(ds["principal"], [[3.0 / 8, 2.0 / 6]] * 3)  # file-level cx / cy do not reach the images
    m = np.asarray(frames[2]["transform_matrix"], np.float32)[:3]
    exp = m.copy()
    exp[:, 3] = exp[:, 3] * np.float32(0.5) + np.float32([0.4, 0.5, 0.6])  # from_na: the two negations cancel, no cycling
    np.testing.assert_allclose(ds["xforms"][2].reshape(4, 3).T, exp, rtol=1e-6)
    # an explicit box replaces scale and offset
    raw["aabb"] = [[-1, -2, -1], [1, 2, 3]]
    path.write_text(json.dumps(raw))
    ds = loader.load_nerf_dataset(path)
    assert ds["scale"] == pytest.approx(0.25)
    np.testing.assert_allclose(ds["offset"], [0.5, 0.5, 0.25])


def test_transparency_alpha_and_mask_files(tmp_path):
    from PIL import Image
    from neus2_b200 import loader
    path, images, _ = write_scene(tmp_path, extra={"white_transparent": True, "black_transparent": True})
    a = np.zeros((6, 8, 4), np.uint8)
    a[..., 0] = 128
    a[..., 3] = 255
    Image.fromarray(a, "RGBA").save(tmp_path / "images" / "000.png.alpha.png")
    mk = np.zeros((6, 8, 4), np.uint8)
    mk[2, 3, 0] = 255
    Image.fromarray(mk, "RGBA").save(tmp_path / "images" / "dynamic_mask_001.png")
    ds = loader.load_nerf_dataset(path)
    px = ds["pixels"].view(np.uint8).reshape(3, 6, 8, 4)
    assert px[1, 0, 0, 3] == 0 and px[1, 0, 1, 3] == 0 and px[2, 0, 0, 3] == 0  # white and black pixels lose their alpha
    assert px[0, 3, 3, 3] == int(255.0 * (((128 / 255 + 0.055) / 1.055) ** 2.4))  # alpha file: linearised red channel
    assert ds["pixels"][1, 2, 3] == 0x00FF00FF  # masked pixel: the marker colour the sample generator skips
    assert np.array_equal(px[2, 1:], images[2][1:])


def test_errors(tmp_path):
    from neus2_b200 import loader
    with pytest.raises(ValueError):
        loader.load_nerf_dataset([])
    path, _, _ = write_scene(tmp_path)
    raw = json.loads(path.read_text())
    del raw["camera_angle_x"]
    path.write_text(json.dumps(raw))
    with pytest.raises(ValueError, match="fov"):
        loader.load_nerf_dataset(path)
    raw["camera_angle_x"] = 0.7
    raw["k1"] = 0.1
    path.write_text(json.dumps(raw))
    with pytest.raises(NotImplementedError):
        loader.load_nerf_dataset(path)
    raw.pop("k1")
    raw["frames"][1]["file_path"] = "images/missing"
    path.write_text(json.dumps(raw))
    with pytest.raises(FileNotFoundError):
        loader.load_nerf_dataset(path)
    raw["frames"] = []
    path.write_text(json.dumps(raw))
    with pytest.raises(ValueError, match="No training images"):
        loader.load_nerf_dataset(path)


def test_directory_of_per_frame_files_is_a_sequence(tmp_path):
    """A data path that is a directory holds one transforms file per frame of a dynamic sequence: every .json whose name does
    not contain "downsample", sorted by base name (src/testbed_nerf.cu:2957-2989)."""
    from neus2_b200 import loader
    for name in ("frame_010.json", "frame_002.json", "frame_002_downsample.json", "notes.txt", "frame_001.JSON"):
        (tmp_path / name).write_text("{}")
    (tmp_path / "sub.json").mkdir()
    got = [p.split("/")[-1] for p in loader.list_frame_jsons(tmp_path)]
    assert got == ["frame_001.JSON", "frame_002.json", "frame_010.json"]
    assert loader.list_frame_jsons(tmp_path / "frame_010.json") == [str(tmp_path / "frame_010.json")]
    with pytest.raises(ValueError):
        loader.list_frame_jsons(tmp_path / "notes.txt")
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(ValueError):
        loader.list_frame_jsons(empty)


def test_focal_length_bits_are_the_reference_loaders():
    """Known answers taken from ngp::load_nerf itself (the reference's loader run on files with these fields): the conversion from
    camera_angle_x / camera_angle_y to a focal length is single-precision arithmetic, and it is compared bit for bit."""
    from neus2_b200 import loader
    got = [np.float32(loader.fov_to_focal_length(96, loader.radians_to_degrees(0.61))), np.float32(loader.fov_to_focal_length(64, loader.radians_to_degrees(0.47)))]
    assert [int(v.view(np.uint32)) for v in got] == [1125676910, 1124444030]  # 152.46652, 133.65427


def test_up_vector_default_and_sequence_writer(tmp_path):
    from neus2_b200 import loader
    from neus2_b200 import synthetic as S
    path, _, _ = write_scene(tmp_path)
    assert loader.load_nerf_dataset(path)["up"] == [0.0, 1.0, 0.0]  # NerfDataset::up (nerf_loader.h:81)
    scenes = [S.render_sphere_views(2, 16, 12, device="cpu", seed=s) for s in (1, 2)]
    d = S.write_sequence_dataset(scenes, str(tmp_path / "seq"))
    files = loader.list_frame_jsons(d)
    assert [f.split("/")[-1] for f in files] == ["frame_0000.json", "frame_0001.json"]
    for f, sc in zip(files, scenes):
        ds = loader.load_nerf_dataset(f)
        np.testing.assert_array_equal(ds["pixels"], sc["pixels"].numpy().view(np.uint32))
        np.testing.assert_array_equal(ds["xforms"], sc["xforms"].numpy())  # scale 1, offset 0: the matrices come back exactly
        np.testing.assert_allclose(ds["focal"], sc["focal"].numpy(), rtol=1e-7)


def test_loader_equals_the_reference_loader_on_the_golden_case():
    """tests/golden/loader_case: a tiny dataset and what ngp::load_nerf returned for it (written by tests/golden/make_loader_golden.py
    where the reference's loader could run).  Cameras, intrinsics and pixel bytes bit for bit."""
    import os
    from neus2_b200 import loader
    case = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "loader_case")
    t = np.load(os.path.join(case, "expected.npz"))
    ds = loader.load_nerf_dataset(os.path.join(case, "transforms.json"))
    assert int(t["header"][0]) == ds["n_images"] == 2 and (int(t["header"][1]), int(t["header"][2]), int(t["header"][3])) == (16, 12, 1)
    assert int(t["header"][4]) == ds["aabb_scale"] and bool(t["header"][6]) == ds["from_na"] and bool(t["header"][7]) == ds["from_mitsuba"]
    assert np.float32(t["floats"][0]) == np.float32(ds["scale"])
    assert np.array_equal(t["floats"][1:4], np.asarray(ds["offset"], np.float32)) and np.array_equal(t["floats"][4:7], np.asarray(ds["up"], np.float32))
    mine = np.asarray(ds["xforms"], np.float32).reshape(-1, 4, 3).transpose(0, 2, 1).reshape(-1, 12)  # column major -> row major
    assert np.array_equal(mine.view(np.uint32), t["xforms"].view(np.uint32))
    assert np.array_equal(np.asarray(ds["focal"], np.float32).view(np.uint32), t["focal"].view(np.uint32))
    assert np.array_equal(np.asarray(ds["principal"], np.float32).view(np.uint32), t["principal"].view(np.uint32))
    assert np.array_equal(np.ascontiguousarray(ds["pixels"]).view(np.uint8).reshape(-1), t["pixels"])
