"""pytest plugin used when the reference project's own test files are run against this package.

Those tests take a ``mocker`` fixture from pytest-mock, which is not installed here; this module
provides the small part of it they use, on top of ``unittest.mock``.
"""

import sys, types, unittest.mock as um, pytest
pm = types.ModuleType("pytest_mock"); 
class MockerFixture:
    def __init__(self): self._patches=[]; self.patch=self._Patch(self); self.MagicMock=um.MagicMock; self.Mock=um.Mock; self.ANY=um.ANY; self.call=um.call; self.mock_open=um.mock_open; self.PropertyMock=um.PropertyMock; self.AsyncMock=um.AsyncMock; self.sentinel=um.sentinel; self.DEFAULT=um.DEFAULT; self.create_autospec=um.create_autospec; self.NonCallableMagicMock=um.NonCallableMagicMock; self.seal=um.seal
    class _Patch:
        def __init__(self, outer): self.o=outer
        def __call__(self, *a, **k): p=um.patch(*a, **k); m=p.start(); self.o._patches.append(p); return m
        def object(self, *a, **k): p=um.patch.object(*a, **k); m=p.start(); self.o._patches.append(p); return m
        def dict(self, *a, **k): p=um.patch.dict(*a, **k); m=p.start(); self.o._patches.append(p); return m
        def multiple(self, *a, **k): p=um.patch.multiple(*a, **k); m=p.start(); self.o._patches.append(p); return m
    def spy(self, obj, name):
        import inspect
        orig=getattr(obj,name); autospec=inspect.ismethod(orig) or inspect.isfunction(orig)
        def wrapper(*a, **k):
            r=orig(*a, **k); spy_obj.spy_return=r; return r
        p=um.patch.object(obj,name,side_effect=wrapper,autospec=autospec); spy_obj=p.start(); self._patches.append(p); return spy_obj
    def stub(self, name=None): return um.MagicMock(name=name)
    def stopall(self):
        for p in reversed(self._patches):
            try: p.stop()
            except RuntimeError: pass
        self._patches=[]
    def resetall(self): pass
pm.MockerFixture=MockerFixture; sys.modules["pytest_mock"]=pm
@pytest.fixture
def mocker():
    m=MockerFixture(); yield m; m.stopall()


import os

if os.environ.get("MLF_REFSUITE_STANDINS") == "1":
    # adapter test files import megatron / nemo / lightning at module level; none is installed here
    import megatron_standins

    megatron_standins.install()
    megatron_standins.install_nemo()

if os.environ.get("MLF_REFSUITE_HOST_ENGINE") == "1":
    # The saver's host logic (bucketing, naming, offsets, results, error paths) with the byte moves
    # done by the numpy test double instead of the CUDA engine; for boxes without a GPU.
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import helpers
    from ml_flashpoint.core import gpu_engine

    gpu_engine.set_default_engine(helpers.NumpyCopyEngine())
