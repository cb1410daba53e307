"""pytest plugin used when the reference project's own test files are run against this package.

Those tests take a ``mocker`` fixture from pytest-mock, which is not installed here; this module
provides the part of it they use, on top of ``unittest.mock``. Two environment switches prepare
the process for test files that need more than this package:

``MLF_REFSUITE_STANDINS=1``     registers the stand-in megatron / nemo / lightning modules
``MLF_REFSUITE_HOST_ENGINE=1``  makes the numpy engine double the process-wide copy engine
"""

import inspect
import os
import sys
import types
import unittest.mock as um

import pytest


class MockerFixture:
    """The subset of pytest-mock's ``MockerFixture`` the reference tests call."""

    MagicMock = um.MagicMock
    Mock = um.Mock
    NonCallableMagicMock = um.NonCallableMagicMock
    PropertyMock = um.PropertyMock
    AsyncMock = um.AsyncMock
    ANY = um.ANY
    DEFAULT = um.DEFAULT
    call = um.call
    sentinel = um.sentinel
    mock_open = staticmethod(um.mock_open)
    create_autospec = staticmethod(um.create_autospec)
    seal = staticmethod(um.seal)

    class _Patcher:
        def __init__(self, owner: "MockerFixture"):
            self._owner = owner

        def _start(self, patcher):
            mock = patcher.start()
            self._owner._patches.append(patcher)
            return mock

        def __call__(self, *args, **kwargs):
            return self._start(um.patch(*args, **kwargs))

        def object(self, *args, **kwargs):
            return self._start(um.patch.object(*args, **kwargs))

        def dict(self, *args, **kwargs):
            return self._start(um.patch.dict(*args, **kwargs))

        def multiple(self, *args, **kwargs):
            return self._start(um.patch.multiple(*args, **kwargs))

    def __init__(self):
        self._patches = []
        self.patch = self._Patcher(self)

    def spy(self, obj, name):
        """Replaces ``obj.name`` with a mock that records calls and still runs the original."""
        original = getattr(obj, name)
        autospec = inspect.ismethod(original) or inspect.isfunction(original)

        def run_original(*args, **kwargs):
            result = original(*args, **kwargs)
            spy_mock.spy_return = result
            return result

        spy_mock = self.patch.object(obj, name, side_effect=run_original, autospec=autospec)
        return spy_mock

    def stub(self, name=None):
        return um.MagicMock(name=name)

    def stopall(self):
        for patcher in reversed(self._patches):
            try:
                patcher.stop()
            except RuntimeError:
                pass
        self._patches = []

    def resetall(self):
        pass


_pytest_mock = types.ModuleType("pytest_mock")
_pytest_mock.MockerFixture = MockerFixture
sys.modules["pytest_mock"] = _pytest_mock


@pytest.fixture
def mocker():
    fixture = MockerFixture()
    yield fixture
    fixture.stopall()


if os.environ.get("MLF_REFSUITE_STANDINS") == "1":
    # adapter test files import megatron / nemo / lightning at module level; none is installed here
    import megatron_standins

    megatron_standins.install()
    megatron_standins.install_nemo()

if os.environ.get("MLF_REFSUITE_HOST_ENGINE") == "1":
    # The saver's host logic (bucketing, naming, offsets, results, error paths) with the byte moves
    # done by the numpy test double instead of the CUDA engine; for boxes without a GPU.
    _tests_dir = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(os.path.dirname(_tests_dir), "oracle"))
    sys.path.insert(0, _tests_dir)
    import helpers
    from ml_flashpoint.core import gpu_engine

    gpu_engine.set_default_engine(helpers.NumpyCopyEngine())
