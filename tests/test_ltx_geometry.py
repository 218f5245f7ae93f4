import numpy as np
import pytest

from solarwm_b200.backends.ltx25 import geometry as geo
from solarwm_b200.errors import BackendContractError


def test_the_stable_geometry_and_its_camera_alignment():
    g = geo.STABLE
    assert g.latent_shape == (128, 20, 16, 24) and g.video_tokens == 20 * 384 and g.first_frame_latent_shape == (128, 1, 16, 24)
    assert g.camera_pixel_indices == (0, 1, 9, 17, 25, 33, 41, 49, 57, 65, 73, 81, 89, 97, 105, 113, 121, 129, 137, 145)
    assert geo.latent_frames_of(81, 4) == 21
    for bad in ((152, 512, 768), (153, 480, 768)):
        with pytest.raises(BackendContractError):
            geo.ClipGeometry(*bad)
    with pytest.raises(BackendContractError):
        geo.latent_frames_of(150)
    poses = np.arange(153 * 16, dtype=np.float64).reshape(153, 4, 4)
    picked = geo.window_cameras(poses)
    assert picked.shape == (20, 4, 4) and picked[2, 0, 0] == 9 * 16
    with pytest.raises(BackendContractError):
        geo.window_cameras(poses[:100])


def test_cover_resize_and_intrinsics_follow_each_other():
    wide = geo.cover_resize(1080, 1920)                                    # 16:9 source into 3:2
    assert (wide.resized_height, wide.resized_width, wide.crop_top, wide.crop_left) == (512, 910, 0, 71)
    tall = geo.cover_resize(1920, 1080)
    assert (tall.resized_height, tall.resized_width, tall.crop_top, tall.crop_left) == (1365, 768, 426, 0)
    k = np.array([[1000.0, 0, 960.0], [0, 1000.0, 540.0], [0, 0, 1]])
    out = geo.transform_intrinsics(k, wide)
    s = 910 / 1920
    assert np.allclose(out, [[1000 * s / 768, 0, (960 * s - 71) / 768], [0, 1000 * (512 / 1080) / 512, 540 * (512 / 1080) / 512], [0, 0, 1]], atol=1e-6)
    normalised = np.array([[1000 / 1920, 0, 0.5], [0, 1000 / 1080, 0.5], [0, 0, 1]])
    assert np.allclose(geo.transform_intrinsics(normalised, wide), out, atol=1e-6)                 # detected as normalised
    assert not np.allclose(geo.transform_intrinsics(normalised, wide, input_normalized=False), out)
    for bad in (np.eye(4), np.array([[1.0, 0.1, 0], [0, 1, 0], [0, 0, 1]]), np.array([[1.0, 0, 0], [0, 1, 0], [0, 0, 2]]),
                np.array([[-1.0, 0, 0], [0, 1, 0], [0, 0, 1]])):
        with pytest.raises(BackendContractError):
            geo.transform_intrinsics(bad, wide)


def test_windows_are_153_consecutive_ordinals():
    ok = np.arange(40, 193, dtype=np.int64)
    assert geo.check_window(ok, start=40) is not None
    for bad in (ok[:-1], ok.astype(np.int32), np.concatenate([ok[:50], ok[51:], ok[-1:] + 1]), ok - 100):
        with pytest.raises(BackendContractError):
            geo.check_window(bad)
    with pytest.raises(BackendContractError):
        geo.check_window(ok, start=41)
