"""The VLM judge client: contact sheets, the strict answer parser, retries, and resumable answers (fake transport)."""
import json

import numpy as np
import pytest

from solarwm_b200.eval.benchmark import Case, judge_pairs, net_preference
from solarwm_b200.eval.judge_client import (HTTPJudge, JudgeAnswerError, JudgeTransportError, QUESTIONS, RecordedJudge, build_prompt,
                                            contact_sheet, parse_answer, sheet_indices)

QS = list(QUESTIONS)


def _clip(level, frames=12, h=18, w=32):
    out = np.zeros((frames, h, w, 3), np.uint8)
    out[..., 0] = level
    out[..., 1] = np.arange(frames, dtype=np.uint8)[:, None, None] * 10
    return out


def test_sheet_indices_and_layout():
    assert sheet_indices(5, 8) == (0, 1, 2, 3, 4)
    assert sheet_indices(81, 8)[0] == 0 and sheet_indices(81, 8)[-1] == 80 and len(set(sheet_indices(81, 8))) == 8
    assert sheet_indices(9, 1) == (0,)
    with pytest.raises(ValueError):
        sheet_indices(0, 4)
    sheet = contact_sheet(_clip(7), cells=6, columns=4, cell_width=16)
    assert sheet.shape == (2 * 9, 4 * 16, 3)
    picks = sheet_indices(12, 6)
    assert int(sheet[0, 0, 1]) == picks[0] * 10 and int(sheet[9, 16, 1]) == picks[5] * 10
    assert sheet[9:, 32:].max() == 0                        # unused cells stay black
    with pytest.raises(ValueError):
        contact_sheet(_clip(1).astype(np.float32))


def test_parser_is_strict():
    text = 'Sure. {"q1_visual_quality": "a", "q4_overall": " Tie ", "note": "{x}"} trailing'
    assert parse_answer(text, ["q1_visual_quality", "q4_overall"]) == {"q1_visual_quality": "A", "q4_overall": "tie"}
    for bad in ("no json", '{"q1_visual_quality": "C"}', '{"q1_visual_quality": 1}', '{"q4_overall": "A"}', '{"q1_visual_quality": "A"'):
        with pytest.raises(JudgeAnswerError):
            parse_answer(bad, ["q1_visual_quality"])
    with pytest.raises(KeyError):
        build_prompt("p", ["q9"], 8)
    assert all(q in build_prompt("a red car", QS, 8) for q in QS)


class FakeEndpoint:
    """Prefers the brighter render; ``script`` is a list of statuses / texts served before it starts answering."""

    def __init__(self, script=()):
        self.script, self.bodies = list(script), []

    def __call__(self, url, headers, body):
        self.url, self.headers = url, headers
        doc = json.loads(body)
        self.bodies.append(doc)
        if self.script:
            step = self.script.pop(0)
            if isinstance(step, int):
                return step, b"busy"
            return 200, json.dumps({"choices": [{"message": {"content": step}}]}).encode()
        import base64, io
        from PIL import Image
        images = [p["image_url"]["url"] for p in doc["messages"][0]["content"] if p["type"] == "image_url"]
        level = [int(np.asarray(Image.open(io.BytesIO(base64.b64decode(u.split(",", 1)[1]))))[0, 0, 0]) for u in images[2:]]
        pick = "tie" if level[0] == level[1] else ("A" if level[0] > level[1] else "B")
        return 200, json.dumps({"choices": [{"message": {"content": json.dumps({q: pick for q in QS})}}]}).encode()


def _judge(endpoint, clips, **kw):
    return HTTPJudge("http://judge.local/v1", "vlm", api_key="k", transport=endpoint, sleep=lambda s: kw.setdefault("slept", []).append(s),
                     frames_of=lambda p: clips[p], image_of=lambda p: clips["structure"][0], first_delay=1.0, **{k: v for k, v in kw.items() if k != "slept"})


def test_request_shape_retries_and_failures():
    clips = {"structure": _clip(5), "a.mp4": _clip(200), "b.mp4": _clip(40)}
    case = Case("hard", "c1", "a red car", "structure", "first.png", None)
    slept = []
    endpoint = FakeEndpoint([429, 503, "not json at all"])
    judge = HTTPJudge("http://judge.local/v1/", "vlm", api_key="k", transport=endpoint, sleep=slept.append, first_delay=1.0,
                      frames_of=lambda p: clips[p], image_of=lambda p: clips["structure"][0])
    assert judge(case, "a.mp4", "b.mp4", QS) == {q: "A" for q in QS}
    assert slept == [1.0, 2.0, 4.0] and judge.requests == 4
    assert endpoint.url == "http://judge.local/v1/chat/completions" and endpoint.headers["Authorization"] == "Bearer k"
    body = endpoint.bodies[-1]
    assert body["temperature"] == 0 and body["model"] == "vlm"
    assert [p["type"] for p in body["messages"][0]["content"]] == ["text"] + ["image_url"] * 4
    assert judge(case, "b.mp4", "a.mp4", QS) == {q: "B" for q in QS}
    with pytest.raises(JudgeTransportError) as err:
        _judge(FakeEndpoint([401]), clips)(case, "a.mp4", "b.mp4", QS)
    assert err.value.status == 401
    with pytest.raises(JudgeTransportError):
        _judge(FakeEndpoint([500, 500]), clips, attempts=2)(case, "a.mp4", "b.mp4", QS)
    with pytest.raises(JudgeAnswerError):
        _judge(FakeEndpoint(["{}", "{}"]), clips, attempts=2)(case, "a.mp4", "b.mp4", QS)


def test_recorded_answers_resume_and_follow_the_files(tmp_path):
    renders = {}
    for method, level in (("ours", 200), ("base", 40)):
        for cid in ("c1", "c2", "c3"):
            path = tmp_path / method / "hard" / f"{cid}.mp4"
            path.parent.mkdir(parents=True, exist_ok=True)
            path.write_bytes(f"{method}-{cid}".encode())
            renders[str(path)] = _clip(level if cid != "c3" else 90)
    renders["structure"] = _clip(5)
    cases = [Case("hard", c, "p", "structure", "f.png", None) for c in ("c1", "c2", "c3")]
    endpoint = FakeEndpoint()
    live = HTTPJudge("http://j/v1", "vlm", transport=endpoint, frames_of=lambda p: renders[p], image_of=lambda p: renders["structure"][0])
    log = tmp_path / "judge" / "answers.jsonl"
    first = RecordedJudge(live, log, judge_id="vlm")
    rows = judge_pairs(cases, tmp_path / "ours", tmp_path / "base", first, QS, a="ours", b="base")
    assert [r["q4_overall"] for r in rows] == ["ours", "ours", "tie"] and first.asked == 6 and first.reused == 0
    stats = net_preference(rows, "q4_overall", a="ours", b="base")
    assert stats["wins"] == 2 and stats["ties"] == 1

    with log.open("a") as fh:                                # an append that was cut short
        fh.write('{"key": "deadbeef", "answ')
    again = RecordedJudge(live, log, judge_id="vlm")
    assert judge_pairs(cases, tmp_path / "ours", tmp_path / "base", again, QS, a="ours", b="base") == rows
    assert again.asked == 0 and again.reused == 6 and len(endpoint.bodies) == 6

    (tmp_path / "ours" / "hard" / "c2.mp4").write_bytes(b"a new render")        # a replaced render is asked again
    third = RecordedJudge(live, log, judge_id="vlm")
    judge_pairs(cases, tmp_path / "ours", tmp_path / "base", third, QS, a="ours", b="base")
    assert third.asked == 2 and third.reused == 4
    assert len(RecordedJudge(live, log, judge_id="vlm").known) == 8
    assert RecordedJudge(live, log, judge_id="other").known.keys() == third.known.keys()   # same file, keys differ per judge id
    lines = log.read_text().splitlines()
    lines[1] = "garbage"
    log.write_text("\n".join(lines) + "\n")
    with pytest.raises(ValueError):
        RecordedJudge(live, log)


def test_command_line_against_a_local_endpoint(tmp_path, capsys):
    """The whole pass over real files and a real HTTP round trip to a server on the loopback interface."""
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer

    from PIL import Image

    from solarwm_b200.eval.judge_client import main
    from solarwm_b200.eval.render_benchmark import write_video

    root = tmp_path / "bench"
    (root / "benchmark" / "hard").mkdir(parents=True)
    (root / "benchmark" / "heldout").mkdir(parents=True)
    rows = []
    for cid in ("s1__day", "s1__night", "s2__day"):
        base = root / "cases" / cid
        base.mkdir(parents=True)
        (base / "prompt.txt").write_text("a street")
        write_video(base / "condition.mp4", _clip(5, frames=9, h=32, w=48))
        Image.fromarray(_clip(5, h=32, w=48)[0]).save(base / "first_frame.png")
        rows.append({"case_id": cid, "files": {k: f"cases/{cid}/{k}" for k in ("prompt.txt", "condition.mp4", "first_frame.png")}})
        write_video(tmp_path / "ours" / "hard" / f"{cid}.mp4", _clip(220, frames=9, h=32, w=48))
        write_video(tmp_path / "base" / "hard" / f"{cid}.mp4", _clip(30, frames=9, h=32, w=48))
    (root / "benchmark" / "hard" / "cases.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    (root / "benchmark" / "heldout" / "cases.jsonl").write_text("")

    brain, seen = FakeEndpoint(), []

    class Handler(BaseHTTPRequestHandler):
        def do_POST(self):
            body = self.rfile.read(int(self.headers["Content-Length"]))
            seen.append((self.path, self.headers.get("Authorization")))
            status, reply = brain(self.path, dict(self.headers), body)
            self.send_response(status)
            self.send_header("Content-Length", str(len(reply)))
            self.end_headers()
            self.wfile.write(reply)

        def log_message(self, *a):
            pass

    server = HTTPServer(("127.0.0.1", 0), Handler)
    thread = threading.Thread(target=server.serve_forever, daemon=True)
    thread.start()
    try:
        argv = ["--root", str(root), "--a", f"ours={tmp_path / 'ours'}", "--b", f"base={tmp_path / 'base'}", "--endpoint",
                f"http://127.0.0.1:{server.server_port}/v1", "--model", "vlm", "--out", str(tmp_path / "out"), "--split", "hard",
                "--questions", "q1_visual_quality,q4_overall", "--cells", "4"]
        assert main(argv) == 0
        first = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert first == {"cases": 3, "asked": 6, "reused": 0, "q1_visual_quality": 1.0, "q4_overall": 1.0}
        assert main(argv) == 0
        assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["reused"] == 6 and len(seen) == 6
    finally:
        server.shutdown()
        server.server_close()
    assert all(path == "/v1/chat/completions" and auth is None for path, auth in seen)
    report = json.loads((tmp_path / "out" / "verdicts-ours-vs-base.json").read_text())
    assert report["net"]["q4_overall"]["wins"] == 3 and [r["case"] for r in report["rows"]] == [f"hard/{r['case_id']}" for r in rows]
