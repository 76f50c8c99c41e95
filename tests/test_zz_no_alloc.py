"""neus2b_generate_samples_static is for hosts that cannot give the library scratch memory (their own allocator owns
the device, or allocation is forbidden once they run): its scratch is built into the library.  It must produce exactly
what neus2b_generate_samples produces, also when called twice in a row on the shared scratch, and it must refuse more
rays than the built-in scratch holds.  Collected last on purpose (file name), and self-contained so it also passes when
run alone in a fresh process."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(oracle):
    from neus2_b200 import _lib as L
    from neus2_b200 import ops
    from neus2_b200 import synthetic as S
    L.lib()
    sc = S.render_sphere_views(6, 80, 80, device="cpu", seed=4)
    ds = ops.make_dataset(sc["pixels"].cuda(), sc["xforms"].cuda(), sc["focal"].cuda(), sc["principal"].cuda())
    # occupancy bits of a solid ball, from the oracle's bitfield builder
    idx = np.arange(128 ** 3, dtype=np.uint32)

    def inv(x):
        x = x & 0x49249249
        x = (x | (x >> 2)) & 0xc30c30c3
        x = (x | (x >> 4)) & 0x0f00f00f
        x = (x | (x >> 8)) & 0xff0000ff
        x = (x | (x >> 16)) & 0x0000ffff
        return x
    c = np.stack([inv(idx), inv(idx >> 1), inv(idx >> 2)], 1).astype(np.float32)
    grid = (np.linalg.norm((c + 0.5) / 128.0 - 0.5, axis=1) < 0.33).astype(np.float32)
    bits, _ = oracle.occ_bitfield(grid, 1)
    ods = oracle.make_dataset(sc["pixels"].numpy().view(np.uint32), sc["xforms"].numpy(), sc["focal"].numpy(), sc["principal"].numpy())
    return L, ops, ds, torch.from_numpy(bits).cuda(), ods, bits


def test_static_scratch_entry_point_matches_the_allocating_one(oracle):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    L, ops, ds, bitfield, ods, bits_host = _setup(oracle)
    cfg = L.train_cfg()
    max_samples = 1 << 19
    for call, (n_rays, total, seed) in enumerate([(8192, 111, 7), (3000, 99999, 8)]):  # two calls in a row, shared scratch
        batch = ops.RayBatch(n_rays, max_samples)
        ops.generate_samples(ds, cfg, n_rays, total, L.pcg32(seed), bitfield, batch)
        i32, f32 = torch.int32, torch.float32
        ray_indices = torch.zeros(n_rays, dtype=i32, device="cuda")
        rays = torch.zeros((n_rays, 6), dtype=f32, device="cuda")
        numsteps = torch.zeros((n_rays, 2), dtype=i32, device="cuda")
        coords = torch.zeros((max_samples, 7), dtype=f32, device="cuda")
        counters = torch.full((8,), -1, dtype=i32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        ops.generate_samples_static(ds, cfg, n_rays, total, L.pcg32(seed), bitfield, max_samples, ray_indices, rays, numsteps,
                                    coords, counters)
        torch.cuda.synchronize()
        if call > 0:  # (the first call on a device looks the scratch arrays' addresses up, which may load the module)
            assert torch.cuda.mem_get_info()[0] == free_before, "the call must not change the device's free memory"
        cnt = batch.counters.cpu().numpy()
        assert cnt[0] > 0 and cnt[1] > 0, "the case must generate samples"
        assert np.array_equal(counters.cpu().numpy(), cnt), call
        k, used = int(cnt[0]), int(cnt[4])
        # integer / index work: bit-exact, the tolerance the other sample-generation tests use
        assert torch.equal(ray_indices[:k], batch.ray_indices[:k])
        assert torch.equal(numsteps[:k], batch.numsteps[:k])
        assert torch.equal(rays[:k].view(i32), batch.rays[:k].view(i32))
        assert torch.equal(coords[:used].view(i32), batch.coords[:used].view(i32))
        # and directly against the CPU restatement of the reference's generator
        ref = oracle.generate_samples(ods, oracle.train_cfg(), n_rays, total, max_samples, oracle.pcg32(seed), bits_host)
        assert k == ref["n_kept"] and int(cnt[1]) == ref["n_samples"]
        assert np.array_equal(numsteps.cpu().numpy().view(np.uint32)[:k], ref["numsteps"][:k])
        assert np.array_equal(coords.cpu().numpy()[:used].view(np.uint32), ref["coords"][:used].view(np.uint32))


def test_static_scratch_entry_point_rejects_oversized_batches(oracle):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    L, ops, ds, bitfield, _, _ = _setup(oracle)
    one = torch.zeros(64, dtype=torch.int32, device="cuda")
    with pytest.raises(L.Neus2bError, match="-5"):
        ops.generate_samples_static(ds, L.train_cfg(), 65537, 0, L.pcg32(1), bitfield, 1024, one, one.float(), one, one.float(), one)
