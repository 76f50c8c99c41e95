"""A scene written to disk in the reference's dataset format (transforms.json + PNG images) goes through the loader into the
testbed and trains like the same scene handed over as arrays."""
import json

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_train_from_a_transforms_file(tmp_path):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from PIL import Image
    from neus2_b200 import _lib as L
    from neus2_b200 import loader
    from neus2_b200 import synthetic as S
    from neus2_b200.testbed import Testbed
    res, n = 96, 10
    sc = S.render_sphere_views(n, res, res, device="cpu", seed=0)
    px = sc["pixels"].numpy().view(np.uint32)
    frames = []
    for i in range(n):
        Image.fromarray(px[i].view(np.uint8).reshape(res, res, 4), "RGBA").save(tmp_path / f"{i:03d}.png")
        X = sc["xforms"][i].numpy()
        ngp = np.stack([X[0:3], X[3:6], X[6:9], X[9:12]], 1)
        nerf = loader.ngp_matrix_to_nerf(ngp, loader.NERF_SCALE, [0.5, 0.5, 0.5])
        frames.append({"file_path": f"{i:03d}", "transform_matrix": np.vstack([nerf, [0, 0, 0, 1]]).tolist()})
    fov = 2.0 * np.arctan(0.5 * res / float(sc["focal"][0, 0]))
    (tmp_path / "transforms.json").write_text(json.dumps({"camera_angle_x": float(fov), "aabb_scale": 1, "frames": frames}))

    tb = Testbed(batch_size=1 << 16)
    ds = tb.load_training_data_from_json(tmp_path / "transforms.json")
    np.testing.assert_array_equal(ds["pixels"], px)
    np.testing.assert_allclose(ds["xforms"], sc["xforms"].numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(ds["focal"], sc["focal"].numpy(), rtol=1e-5)
    tb.set_params(S.init_params(L.grid_n_params(tb.config.grid), seed=1337))
    first = tb.train(1).loss
    last = tb.train(250).loss
    assert np.isfinite(last) and last < 0.2 * first
    # a camera given in the dataset's convention renders the object in the middle of the picture
    X = sc["xforms"][3].numpy()
    tb.set_nerf_camera_matrix(loader.ngp_matrix_to_nerf(np.stack([X[0:3], X[3:6], X[6:9], X[9:12]], 1), ds["scale"], ds["offset"]))
    tb.fov = float(np.degrees(fov))
    tb.background_color = [0.0, 0.0, 0.0, 0.0]  # (the default background is opaque black)
    img = tb.render(64, 64)
    assert img[24:40, 24:40, 3].mean() > 0.9 and img[:4, :4, 3].mean() < 0.1
    tb.close()
    with pytest.raises(ValueError):
        Testbed(batch_size=1 << 16, n_cascades=2).load_training_data_from_json(tmp_path / "transforms.json")
