"""``jax_plugins.qmm_b200.initialize()`` against a stand-in for jax's ``xla_bridge`` (jax is not
installed here): library discovery, the GetPjrtApi check, the register_plugin call with the
reference's arguments (src/jax_plugins/silicon/__init__.py:195-200) and the entry-point metadata."""

import os
import subprocess
import sys
import types

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture
def plugin(monkeypatch):
    import jax_plugins.qmm_b200 as plugin

    return plugin


def _fake_jax(monkeypatch, with_register=True):
    calls = []
    jax = types.ModuleType("jax")
    jax.config = types.SimpleNamespace(update=lambda k, v: calls.append(("config", k, v)))
    src = types.ModuleType("jax._src")
    xb = types.ModuleType("jax._src.xla_bridge")
    xb._backends = {}
    if with_register:
        xb.register_plugin = lambda name, **kw: calls.append(("register", name, kw))
    src.xla_bridge = xb
    jax._src = src
    monkeypatch.setitem(sys.modules, "jax", jax)
    monkeypatch.setitem(sys.modules, "jax._src", src)
    monkeypatch.setitem(sys.modules, "jax._src.xla_bridge", xb)
    return calls


def test_library_discovery_and_env_override(plugin, monkeypatch, tmp_path):
    found = plugin.find_library()
    assert found is not None and found.endswith("libqmm.so")
    other = tmp_path / "libqmm.so"
    other.write_bytes(b"")
    monkeypatch.setenv("QMM_LIBRARY_PATH", str(other))
    assert plugin.find_library() == str(other)
    monkeypatch.setenv("QMM_LIBRARY_PATH", str(tmp_path / "missing.so"))
    with pytest.warns(UserWarning):
        assert plugin.find_library() == found  # falls back to the search paths


def test_initialize_says_when_the_pjrt_table_is_not_built(plugin, monkeypatch):
    _fake_jax(monkeypatch)
    lib = plugin.find_library()
    if plugin.exports_pjrt_api(lib):
        pytest.skip("this build has the PJRT table")
    with pytest.raises(plugin.QmmPluginError) as e:
        plugin.initialize()
    assert "GetPjrtApi" in str(e.value) and "pjrt_c_api.h" in str(e.value)


def test_initialize_registers_the_backend_like_the_reference(plugin, monkeypatch):
    calls = _fake_jax(monkeypatch)
    monkeypatch.setattr(plugin, "exports_pjrt_api", lambda path: True)  # as if built with the table
    plugin.initialize()
    assert ("config", "jax_use_shardy_partitioner", False) in calls
    reg = [c for c in calls if c[0] == "register"]
    assert len(reg) == 1 and reg[0][1] == "qmm_b200"
    assert reg[0][2]["priority"] == 500 and reg[0][2]["options"] == {}
    assert reg[0][2]["library_path"].endswith("libqmm.so")


def test_initialize_errors(plugin, monkeypatch):
    _fake_jax(monkeypatch, with_register=False)
    monkeypatch.setattr(plugin, "exports_pjrt_api", lambda path: True)
    with pytest.raises(plugin.QmmPluginError) as e:
        plugin.initialize()
    assert "register_plugin" in str(e.value)
    monkeypatch.setattr(plugin, "find_library", lambda: None)
    with pytest.raises(plugin.QmmPluginError) as e:
        plugin.initialize()
    assert "Could not find libqmm.so" in str(e.value)


def test_entry_point_metadata():
    import tomllib

    meta = tomllib.load(open(os.path.join(ROOT, "pyproject.toml"), "rb"))
    assert meta["project"]["entry-points"]["jax_plugins"] == {"qmm_b200": "jax_plugins.qmm_b200"}
    # the module the entry point names imports without jax and exposes initialize()
    out = subprocess.run([sys.executable, "-c", "import jax_plugins.qmm_b200 as p; print(callable(p.initialize))"],
                         cwd=ROOT, capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "True", out.stderr
