import json
import urllib.request

import numpy as np
import pytest

from solarwm_b200.serve import camera_control as cc
from solarwm_b200.serve.state import SessionState
from solarwm_b200.serve.web import make_server, serve_in_thread


def test_action_strings_and_padding():
    acts = cc.parse_action_string("w-2, dl-1，none-1")
    assert acts == [["w"], ["w"], ["d", "l"], []]
    assert cc.fit_action_steps(acts, num_transitions=6)[-1] == []
    for bad in ("", "w", "w-0", "x-1", "w-1,,a-1", "-2"):
        with pytest.raises(ValueError):
            cc.parse_action_string(bad)
    with pytest.raises(ValueError):
        cc.fit_action_steps(acts, num_transitions=3)


def test_camera_integration_is_smooth_and_bounded():
    st = cc.KeyboardCameraState(cc.KeyboardCameraConfig(acceleration_seconds=0.25))
    z = [st.step("w")[2, 3] for _ in range(16)]
    steps = np.diff([0.0] + z)
    assert np.all(steps[1:] >= steps[:-1] - 1e-6) and abs(steps[-1] - 1.2 / 16) < 1e-6      # accelerates to full speed
    assert abs(steps[0] - (1.2 / 16) / 4) < 1e-6
    coast = [st.step([])[2, 3] for _ in range(8)]
    assert coast[-1] == pytest.approx(coast[-2])                                             # decelerates to rest
    st = cc.KeyboardCameraState(cc.KeyboardCameraConfig(acceleration_seconds=0.0, pitch_speed_degrees_per_second=600))
    for _ in range(16):
        st.step("i")
    assert st.pitch == pytest.approx(np.radians(85.0))
    R = st.c2w[:3, :3]
    assert np.allclose(R @ R.T, np.eye(3), atol=1e-9)
    poses = cc.actions_to_latent_c2w(cc.parse_action_string("l-3"), temporal_stride=4)
    assert poses.shape == (4, 4, 4) and np.allclose(poses[0], np.eye(4))
    with pytest.raises(ValueError):
        st.set_move_speed_scale(10.0)


def test_web_state_and_keys():
    state, nav = SessionState(), cc.NavigationState()
    server = make_server(state, nav, port=0)
    serve_in_thread(server)
    base = f"http://127.0.0.1:{server.server_address[1]}"

    def post(path, payload):
        req = urllib.request.Request(base + path, data=json.dumps(payload).encode(), method="POST")
        try:
            return urllib.request.urlopen(req).status
        except urllib.error.HTTPError as e:
            return e.code

    page = urllib.request.urlopen(base + "/")
    html = page.read().decode()
    assert page.headers["Content-Type"].startswith("text/html") and "/key" in html and "/state" in html and "wasdijkl" in html
    assert post("/key", {"key": "w", "down": True}) == 200 and nav.down == {"w"}
    assert post("/key", {"key": "q", "down": True}) == 400
    assert post("/command", {"op": "start"}) == 200 and state.next_command()["op"] == "start"
    assert post("/command", {"op": "explode"}) == 400
    state.generated(0, 12.5, 3.0)
    snap = json.loads(urllib.request.urlopen(base + "/state").read())
    assert snap["chunks"] == 1 and snap["recent"][0]["dit_ms"] == 12.5
    server.shutdown()


def test_worker_smoke_on_cpu(tmp_path, capsys):
    from solarwm_b200.serve.worker import main

    assert main(["--smoke", "--model", "tiny", "--height", "8", "--width", "8", "--chunk-frames", "1", "--window-frames", "3",
                 "--chunks", "4", "--output", str(tmp_path)]) == 0
    report = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert report["chunks"] == 4
    assert json.loads((tmp_path / "exit-rank0.json").read_text())["status"] == "ok"


def test_memory_retrieval_prefers_overlapping_views_outside_recent_window():
    import numpy as np
    import torch

    from solarwm_b200.serve.memory import LatentMemoryBank, RetrievalCameras, retrieval_scores, select_memory

    K = np.array([[0.5, 0, 0.5], [0, 0.9, 0.5], [0, 0, 1.0]])

    def cam(x=0.0, yaw=0.0):
        c = np.eye(4)
        c[0, 3] = x
        c[:3, :3] = np.array([[np.cos(yaw), 0, np.sin(yaw)], [0, 1, 0], [-np.sin(yaw), 0, np.cos(yaw)]])
        return c

    q = cam()
    s = retrieval_scores(q, [cam(), cam(x=8.0), cam(yaw=np.pi)], K)
    assert s[0] > s[1] > s[2] and abs(s[0] - 1.0) < 1e-9          # identical view: full overlap, no penalty
    # a walk away and back: at chunk 8 the best memory is the start of the walk, never the recent chunks
    cams = RetrievalCameras()
    xs = list(np.linspace(0, 40, 25)) + list(np.linspace(40, 0, 20))
    for x in xs:
        cams.append(cam(x=float(x)), K)
    idx, sc = cams.select(8)
    assert len(idx) == 5 and idx.max() < (8 - 5) * 5 and list(sc) == sorted(sc, reverse=True)
    assert 0 in idx
    none, _ = select_memory(np.stack(cams.c2w), np.stack(cams.K), 3)
    assert len(none) == 0
    bank = LatentMemoryBank()
    for i in range(3):
        bank.commit(torch.full((1, 2, 5, 2, 2), float(i)), i)
    got = bank.gather([1, 7, 14], torch.zeros(1, 2, 5, 2, 2))
    assert got.shape == (1, 2, 3, 2, 2) and got[0, 0, :, 0, 0].tolist() == [0.0, 1.0, 2.0]


def test_decode_backends_switch_orders_chunks_and_refuses_nonfinite_pixels():
    import pytest
    import torch

    from solarwm_b200.models.vae import StreamingDecoder, VAEConfig, VideoVAE
    from solarwm_b200.models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder
    from solarwm_b200.serve.decode_backends import DecodeBackends, finite_host

    torch.manual_seed(0)
    vcfg = ViTDecoderConfig.tiny()
    vit = ViTVideoDecoder(vcfg, device="cpu", dtype=torch.float32, seed=0)
    vae = VideoVAE(VAEConfig(z_dim=4, base=8, temporal_ups=(True, False), out_channels=3)).eval()
    backends = DecodeBackends({"vit": lambda: StreamingViTDecoder(vit, (4, 6)), "conv": lambda: StreamingDecoder(vae)}, pin=False)
    with pytest.raises(ValueError):
        DecodeBackends({"nope": lambda: None})
    pieces = []
    with pytest.raises(RuntimeError, match="reordered"):
        backends.push(0, torch.zeros(4, 5, 4, 6), lambda *a: pieces.append(a))     # not started
    for kind, first, rest in (("vit", 1, vcfg.frames_per_latent), ("conv", 1, 2)):
        pieces.clear()
        backends.start(kind)
        ms = backends.push(0, torch.randn(4, 5, 4, 6), lambda *a: pieces.append(a))
        assert ms > 0 and [p[1] for p in pieces] == [0, 1, 2, 3, 4] and all(p[0] == 0 for p in pieces)
        assert pieces[0][2].shape[1] == first and pieces[1][2].shape[1] == rest
        assert pieces[1][3] >= pieces[0][3]
        with pytest.raises(RuntimeError, match="reordered"):
            backends.push(5, torch.randn(4, 5, 4, 6), lambda *a: None)
        backends.push(1, torch.randn(4, 5, 4, 6), lambda *a: pieces.append(a))
        assert len(pieces) == 10
        with pytest.raises(FloatingPointError):
            backends.push(2, torch.full((4, 5, 4, 6), float("nan")), lambda *a: None)
        backends.finish()
    assert finite_host(torch.ones(3, dtype=torch.bfloat16)) and not finite_host(torch.tensor([float("inf")], dtype=torch.bfloat16))
    backends.close()


def test_scene_upload_validation_and_isolated_preparation(tmp_path):
    import base64
    import io
    import os
    import threading
    import time

    import pytest
    from PIL import Image

    from solarwm_b200.serve import scene_inputs as si

    def png(w, h, fmt="PNG"):
        buf = io.BytesIO()
        Image.new("RGB", (w, h), (200, 100, 50)).save(buf, format=fmt)
        return base64.b64encode(buf.getvalue()).decode()

    row = si.store_upload(tmp_path, {"prompt": " a quiet street ", "image": png(32, 16)})
    assert row["scene_id"].startswith("upload-") and row["prompt"] == "a quiet street" and os.path.exists(row["first"])
    assert si.store_upload(tmp_path, {"prompt": "a quiet street", "image": png(32, 16)}) == row       # idempotent
    assert si.store_upload(tmp_path, {"prompt": "another", "image": png(32, 16, "JPEG")})["scene_id"] != row["scene_id"]
    for bad in ({"prompt": "", "image": png(4, 4)}, {"prompt": "x", "image": "@@@"}, {"prompt": "x", "image": png(4, 4, "BMP")},
                {"prompt": "x", "image": "A" * (12 * 1024 * 1024)}, {"prompt": "x", "image": png(5000, 4000)},
                {"prompt": "x" * 4001, "image": png(4, 4)}):
        with pytest.raises(ValueError):
            si.store_upload(tmp_path, bad)
    # the conditioning function runs in another process, without the launcher's rank variables
    os.environ["RANK"] = "3"
    try:
        req = {"callable": "solarwm_b200.serve.scene_inputs:image_statistics", "args": [row["first"]]}
        seen = []
        out = si.prepare_isolated(tmp_path, req, progress=seen.append)
    finally:
        del os.environ["RANK"]
    assert out["pid"] != os.getpid() and abs(out["mean"][0] - 200 / 255) < 1e-3 and seen == ["encoding", "encoded"]
    assert si.prepare_isolated(tmp_path, req, progress=seen.append) == out and seen == ["encoding", "encoded"]   # cached
    with pytest.raises(RuntimeError, match="FileNotFoundError"):
        si.prepare_isolated(tmp_path, {"callable": "solarwm_b200.serve.scene_inputs:image_statistics", "args": ["/nonexistent.png"]})
    # cancellation and timeout end the child
    flag = threading.Event()
    threading.Timer(0.3, flag.set).start()
    t0 = time.monotonic()
    with pytest.raises(si.PreparationCancelled):
        si.prepare_isolated(tmp_path, {"callable": "time:sleep", "args": [30]}, cancelled=flag.is_set)
    with pytest.raises(TimeoutError):
        si.prepare_isolated(tmp_path, {"callable": "time:sleep", "args": [31]}, timeout_s=0.3)
    assert time.monotonic() - t0 < 20


def test_worker_decodes_chunks_through_the_decoder_switch(tmp_path, capsys):
    import pytest

    from solarwm_b200.serve.worker import main

    for kind in ("vit", "conv"):
        out = tmp_path / kind
        assert main(["--smoke", "--model", "tiny", "--height", "8", "--width", "8", "--chunk-frames", "1", "--window-frames", "3",
                     "--chunks", "3", "--decoder", kind, "--output", str(out)]) == 0
        report = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert report["decoder"] == kind and report["decoded_frames"] >= 3 and report["median_decode_ms"] > 0
        assert (out / "frames" / "video.rgb").stat().st_size > 0
    with pytest.raises(SystemExit):
        main(["--smoke", "--decoder", "nope"])


def test_worker_h3_family_streams_and_decodes(tmp_path, capsys):
    from solarwm_b200.serve.worker import main

    assert main(["--smoke", "--family", "h3", "--model", "tiny", "--height", "4", "--width", "6", "--chunk-frames", "2",
                 "--window-frames", "4", "--chunks", "4", "--decoder", "vit", "--no-graphs", "--output", str(tmp_path)]) == 0
    report = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert report["family"] == "h3" and report["chunks"] == 4 and report["decoded_frames"] > 0
    assert json.loads((tmp_path / "exit-rank0.json").read_text())["chunks"] == 4
    session = json.loads((tmp_path / "session.json").read_text())
    assert session["schema"] == "solarwm.serve-session.v1" and len(session["chunks"]) == 4 and "dit_ms" in session["chunks"][0]


def test_decode_parity_tool_reports_streaming_equals_one_shot(capsys):
    from solarwm_b200.serve.decode_parity import main

    for kind in ("conv", "vit"):
        assert main(["--decoder", kind, "--frames", "9", "--device", "cpu", "--tolerance", "1e-4"]) == 0
        report = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert report["decoder"] == kind and report["max_abs_diff"] <= 1e-4
