"""pytest plugin used when the reference project's own test files are run against this package.

Those tests take a ``mocker`` fixture from pytest-mock, which is not installed here; this module
provides the small part of it they use, on top of ``unittest.mock``.
"""

import sys, types, unittest.mock as um, pytest
pm = types.ModuleType("pytest_mock"); 
class MockerFixture:
    def __init__(self): self._patches=[]; self.patch=self._Patch(self); self.MagicMock=um.MagicMock; self.Mock=um.Mock; self.ANY=um.ANY; self.call=um.call; self.mock_open=um.mock_open; self.PropertyMock=um.PropertyMock; self.AsyncMock=um.AsyncMock; self.sentinel=um.sentinel; self.DEFAULT=um.DEFAULT
    class _Patch:
        def __init__(self, outer): self.o=outer
        def __call__(self, *a, **k): p=um.patch(*a, **k); m=p.start(); self.o._patches.append(p); return m
        def object(self, *a, **k): p=um.patch.object(*a, **k); m=p.start(); self.o._patches.append(p); return m
        def dict(self, *a, **k): p=um.patch.dict(*a, **k); m=p.start(); self.o._patches.append(p); return m
        def multiple(self, *a, **k): p=um.patch.multiple(*a, **k); m=p.start(); self.o._patches.append(p); return m
    def spy(self, obj, name):
        orig=getattr(obj,name); m=um.MagicMock(side_effect=orig); p=um.patch.object(obj,name,m); p.start(); self._patches.append(p); return m
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
