"""probe_mi_extraction, generate_comparison_visuals and the datasets-server streaming client (against a server on
127.0.0.1 and against file:// pages)."""
import http.server
import json
import os
import subprocess
import sys
import threading
import urllib.parse

import pytest

from transformers_fusion_b200.cli import generate_comparison_visuals as GV, probe_mi_extraction as PM
from transformers_fusion_b200.utils.hf_streamer import HFStreamer, HTTPClient, SimpleJSON

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_probe_rows_and_launcher():
    out, total, mi, ex = PM.probe(["0.4 2.6 0 0.3 1", "1.0 1.2 0 0.9 1", "0.5 0.6 1 0.2 0", "bad"])
    assert (total, mi, ex) == (3, 2, 1)
    assert out[0] == "row=1 gap=2.200 mi=SUSPECT extraction=SUSPECT" and out[1].endswith("mi=OK extraction=OK")
    assert out[-2] == "summary rows=3 mi_suspect=2 extraction_suspect=1"
    r = subprocess.run([os.path.join(ROOT, "bin", "probe_mi_extraction")], input="0.4 2.6 0 0.3 1\n", capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "summary rows=1 mi_suspect=1 extraction_suspect=1" in r.stdout


def test_comparison_visuals(tmp_path):
    csvp, outp = tmp_path / "cmp.csv", tmp_path / "docs" / "charts.md"
    csvp.write_text("dataset,format,bpw,mse,psnr,enc,dec,x\n"
                    "gaussian,Q_8,8,1e-5,50.1,1,1,0\ngaussian,[ref] int4,4,3e-3,25.2,1,1,0\ngaussian,Q_G_4,4,2e-3,27.0,1,1,0\n"
                    "real,MXQ_4,4,1e-3,30.5,1,1,0\nreal,broken,x,y,z\n")
    assert GV.main(["--input", str(csvp), "--output", str(outp)]) == 0
    md = outp.read_text()
    assert md.count("<svg") == 2 and md.count("<circle") == 4 and "## Dataset: real" in md
    assert "#d33" in md and "#083" in md and "#c6a700" in md and "| Q_8 | 8 | 1.000e-05 | 50.10 |" in md
    assert GV.main(["--input", str(tmp_path / "missing.csv")]) == 1
    (tmp_path / "empty.csv").write_text("dataset,format,bpw,mse,psnr\n")
    assert GV.main(["--input", str(tmp_path / "empty.csv"), "--output", str(outp)]) == 2


class _Handler(http.server.BaseHTTPRequestHandler):
    ROWS = [{"row": {"text": f"sample {i}"}} for i in range(7)] + [{"row": {"label": 3, "content": "last"}}]

    def log_message(self, *a): pass

    def _send(self, body: bytes, code=200, extra=None):
        self.send_response(code)
        self.send_header("Content-Length", str(len(body)))
        for k, v in (extra or {}).items():
            self.send_header(k, v)
        self.end_headers()
        if self.command != "HEAD":
            self.wfile.write(body)

    def do_HEAD(self): self._send(b"x" * 100)

    def do_GET(self):
        u = urllib.parse.urlparse(self.path)
        q = urllib.parse.parse_qs(u.query)
        if u.path == "/rows":
            if self.headers.get("Authorization") != "Bearer tok":
                return self._send(b"{}", 401)
            off, n = int(q["offset"][0]), int(q["length"][0])
            if q["dataset"][0] != "org/data":
                return self._send(b'{"error": "not found"}', 404)
            self._send(json.dumps({"rows": self.ROWS[off:off + n], "num_rows_total": len(self.ROWS)}).encode())
        elif u.path == "/blob":
            data = bytes(range(100))
            rng = self.headers.get("Range")
            if rng:
                a, b = (int(x) for x in rng.split("=")[1].split("-"))
                return self._send(data[a:b + 1], 206)
            self._send(data)
        else:
            self._send(b"", 404)


def test_streamer_against_local_server_and_files(tmp_path):
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _Handler)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{srv.server_port}"
    try:
        http_ = HTTPClient(5)
        assert http_.range_request(base, "/blob", 10, 19) == bytes(range(10, 20))
        assert http_.get_content_length(base, "/blob") == 100 and len(http_.get_binary(base, "/blob")) == 100
        st = HFStreamer(base, page=3, client=http_)
        assert not st.open("org/data") and "401" in st.last_error          # no token
        http_.set_auth_token("tok")
        assert st.open("org/data", "train") and st.is_open()
        got = list(st)
        assert got == [f"sample {i}" for i in range(7)] + ["last"] and st.samples_streamed() == 8
        st.close()
        assert not st.is_open() and st.next_sample() is None
        assert not HFStreamer(base, client=http_).open("org/none")
    finally:
        srv.shutdown()
    d = tmp_path / "pages"
    d.mkdir()
    (d / "a__b.train.0.json").write_text(json.dumps({"rows": [{"row": {"text": "x"}}, {"row": {"text": "y"}}]}))
    (d / "a__b.train.2.json").write_text(json.dumps({"rows": [{"row": {"text": "z"}}]}))
    fs = HFStreamer("file://" + str(d), page=2)
    assert fs.open("a/b") and list(fs) == ["x", "y", "z"]
    assert SimpleJSON.find_all_rfilenames(SimpleJSON.find_array('{"siblings": [{"rfilename": "a.bin"}, {"x": 1}]}', "siblings")) == ["a.bin"]
    assert SimpleJSON.url_encode("a b/c") == "a%20b%2Fc" and SimpleJSON.escape('q"') == 'q\\"'
