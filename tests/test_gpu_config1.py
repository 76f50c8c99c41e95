"""BASELINE config 1 over its whole schedule: 64 views 512 x 512 of the analytic sphere, hash grid 16 levels x 2 features
(scale 1.447, T = 2^19), batch 2^18 samples, eikonal weight 0.1, Adam at 1e-2, 2 000 steps.

Everything the config does not name stays at what the reference ships for static scenes (configs/nerf/dtu.json), which
includes the progressive level mask (base_training_step 200, valid_level_scale 0.02, base_valid_level_scale 0.2): the
reference applies it to every run.  Without the mask this combination (eikonal 0.1 on levels up to resolution 4 000 at a
learning rate of 1e-2) destabilises between steps 1 300 and 2 900; the second case shows the same 16 levels staying stable
with the reference's own eikonal weight 0.01 and no mask."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DTU_MASK = dict(base_training_step=200, valid_level_scale=0.02, base_valid_level_scale=0.2)


@pytest.fixture(scope="module")
def scene():
    from neus2_b200 import synthetic as S
    s = S.render_sphere_views(64, 512, 512, fov_deg=40.0, radius=0.3, seed=0, device="cuda")
    return {k: (v.cpu().numpy() if hasattr(v, "cpu") else v) for k, v in s.items()}


@pytest.mark.parametrize("name,kw", [("config1", dict(ek_loss_weight=0.1, **DTU_MASK)), ("eikonal_0.01_unmasked", dict(ek_loss_weight=0.01))])
def test_config1_trains_through_its_schedule(scene, name, kw):
    from neus2_b200 import _lib as L
    from neus2_b200 import synthetic as S
    from neus2_b200.parallel import device_view
    from neus2_b200.testbed import Testbed
    from util import record
    tb = Testbed(batch_size=1 << 18, learning_rate=1e-2, **kw)
    tb.load_training_data(scene["pixels"], scene["xforms"], scene["focal"], scene["principal"])
    ng = L.grid_n_params(tb.config.grid)
    tb.set_params(S.init_params(ng, seed=1337))
    variance = device_view(tb.device_ptrs()["master"], (12288 + ng + 4) * 4, torch.float32)[12288 + ng:]
    hist = []
    for _ in range(40):
        st = tb.train(50)
        hist.append((st.training_step, st.loss, st.ek_loss, float(variance[0])))
        assert np.isfinite(st.loss) and np.isfinite(st.ek_loss) and st.overflow == 0 and st.nonfinite_gradients == 0, hist[-1]
    assert st.training_step == 2000
    losses = np.array([h[1] for h in hist])
    var = np.array([h[3] for h in hist])
    # the loss of the last quarter stays at the level it reached: no return to the fog
    assert losses[-10:].max() < 2e-4 and losses[-10:].max() < 4 * np.median(losses[20:30]) + 1e-5, hist[-12:]
    # the learned sharpness exp(10 * variance) keeps growing or holds; a collapse shows as a fall below its start (0.3)
    assert var[-10:].min() > 0.5 and var[-1] > 0.9 * var.max(), list(var)
    v, i = tb.compute_marching_cubes_mesh(256, use_ema=True)
    r = np.linalg.norm(v.cpu().numpy() - 0.5, axis=1)
    mean_d, p99 = float(np.abs(r - 0.3).mean()), float(np.quantile(np.abs(r - 0.3), 0.99))
    record("config1_2000_steps_" + name, mean_abs_dist=mean_d, p99=p99, n_verts=int(v.shape[0]), final_loss=float(losses[-1]),
           final_variance=float(var[-1]))
    # one-sided Chamfer distance mesh -> sphere: well under the 0.008 that 600 steps on 12 small views reach
    assert v.shape[0] > 10000 and mean_d < 0.004 and p99 < 0.02, (mean_d, p99)
    tb.close()
