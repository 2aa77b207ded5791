"""The three places that list the library's translation units agree: the build
script, the Rust crate's build.rs and the files under csrc/."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_source_lists_agree():
    csrc = sorted(f for f in os.listdir(os.path.join(ROOT, "oxmera_b200", "csrc")) if f.endswith(".cu"))
    from oxmera_b200 import build
    assert sorted(build.SOURCES) == csrc
    rs = open(os.path.join(ROOT, "rust", "oxmera-b200", "build.rs")).read()
    assert sorted(set(re.findall(r'"([a-z0-9_]+\.cu)"', rs))) == csrc
