"""The kernel build helper, as far as it goes without a GPU or a compiler run."""
from concurrent.futures import ThreadPoolExecutor

from infernum_b200.csrc import build


def test_build_dir_from_many_threads(tmp_path, monkeypatch):
    """Modules are compiled from several threads at once; each of them asks for
    the folder, and none may be sent elsewhere because another one's probe file
    came and went."""
    target = tmp_path / "kernels"
    monkeypatch.setenv("INFERNUM_BUILD_DIR", str(target))
    with ThreadPoolExecutor(max_workers=16) as pool:
        dirs = list(pool.map(lambda _: build.build_dir(), range(300)))
    assert set(dirs) == {str(target)}
    assert [p.name for p in target.iterdir()] == []  # no probe file is left behind


def test_module_hash_follows_sources_and_flags():
    a = build._hash_module(["elementwise.cu"], [], "nvcc")
    assert a == build._hash_module(["elementwise.cu"], [], "nvcc")
    assert a != build._hash_module(["elementwise.cu"], ["-DIB_HD=64"], "nvcc")
    assert a != build._hash_module(["sampling.cu"], [], "nvcc")
