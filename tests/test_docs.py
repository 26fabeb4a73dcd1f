"""The guides stay in step with the code: every environment variable the
package reads is listed in docs/env.md and every variable listed there is
read somewhere; links between guides resolve; the examples the guides name
exist."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE_SUFFIXES = (".py", ".cc", ".cpp", ".h", ".cu", ".cuh")
# build-time switches of the reference's CMake build and names that only look like variables
NOT_VARIABLES = {"HOROVOD_WITH_PYTORCH",
                 "HOROVOD_SECRET_KEY"}  # the Python name of "_HOROVOD_SECRET_KEY", which the guide lists


def _source_text():
    chunks = []
    for base in ("horovod_b200", "bench.py", "bench_collectives.py", "bench_kernels.py"):
        path = os.path.join(ROOT, base)
        if os.path.isfile(path):
            chunks.append(open(path).read())
            continue
        for folder, _dirs, files in os.walk(path):
            for name in files:
                if name.endswith(SOURCE_SUFFIXES):
                    chunks.append(open(os.path.join(folder, name), errors="ignore").read())
    return "\n".join(chunks)


def test_environment_reference_matches_the_code():
    text = _source_text()
    in_code = set(re.findall(r"\bHOROVOD_[A-Z0-9_]+\b", text))
    in_code = {v for v in in_code if not v.endswith(("_H", "_H_"))} - NOT_VARIABLES
    doc = open(os.path.join(ROOT, "docs", "env.md")).read()
    in_doc = set(re.findall(r"\bHOROVOD_[A-Z0-9_]+\b", doc))
    prefixes = {m[:-1] for m in re.findall(r"\bHOROVOD_[A-Z0-9_]+\*", doc)}  # e.g. HOROVOD_LSF_*
    in_doc -= {p.rstrip("_") for p in prefixes}
    missing = sorted(v for v in in_code - in_doc if not any(v.startswith(p) for p in prefixes))
    assert not missing, "read by the code but not in docs/env.md: %s" % missing
    unknown = sorted(v for v in in_doc - in_code if not any(v.startswith(p) for p in prefixes))
    assert not unknown, "in docs/env.md but read nowhere: %s" % unknown


def test_links_and_named_files_in_the_guides_exist():
    docs = os.path.join(ROOT, "docs")
    for name in sorted(os.listdir(docs)):
        if not name.endswith(".md"):
            continue
        body = open(os.path.join(docs, name)).read()
        for target in re.findall(r"\]\(([^)#]+\.md)\)", body):
            assert os.path.exists(os.path.join(docs, target)), "%s links to %s" % (name, target)
        for path in re.findall(r"`((?:examples|docs|tests)/[A-Za-z0-9_./-]+\.(?:py|md))`", body):
            assert os.path.exists(os.path.join(ROOT, path)), "%s names %s" % (name, path)
    readme = open(os.path.join(ROOT, "README.md")).read()
    for path in re.findall(r"`((?:examples|docs|tests|profiles)/[A-Za-z0-9_./-]+\.(?:py|md))`", readme):
        assert os.path.exists(os.path.join(ROOT, path)), "README names %s" % path
