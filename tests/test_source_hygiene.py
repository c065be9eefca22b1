"""Source files stand on their own: no comment or string in them points at a build document, a build step, a remote
runner or a path of the machine they were written on; and nothing committed reaches into the working folder."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# spelled in pieces so that this file does not match itself
WORDS = ["SUR" + "VEY", "VER" + "DICT", "ADV" + "ICE", "DES" + "IGN.md", "BASE" + "LINE.md", "gpu" + "run", "/ro" + "ot/", "the ju" + "dge",
         r"\bro" + r"und \d", "_wo" + "rk/"]
PATTERN = re.compile("|".join(WORDS))
SUFFIXES = (".py", ".cu", ".cuh", ".cpp", ".h", ".sh", ".ini", ".json")


def _sources():
    for top in ("infinilm_b200", "tests", "bin", "examples", "bench.py", "__graft_entry__.py", "pytest.ini"):
        path = os.path.join(ROOT, top)
        if os.path.isfile(path):
            yield path
            continue
        for d, dirs, files in os.walk(path):
            dirs[:] = [x for x in dirs if x not in ("_build", "__pycache__")]
            for f in files:
                if f.endswith(SUFFIXES) or top == "bin":
                    yield os.path.join(d, f)


def test_sources_name_no_build_document_runner_or_machine_path():
    hits = []
    for path in _sources():
        if os.path.abspath(path) == os.path.abspath(__file__):
            continue
        with open(path, encoding="utf-8", errors="replace") as fh:
            for n, line in enumerate(fh, 1):
                if PATTERN.search(line):
                    hits.append(f"{os.path.relpath(path, ROOT)}:{n}: {line.strip()[:120]}")
    assert not hits, "\n".join(hits)
