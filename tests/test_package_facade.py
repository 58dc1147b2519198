"""Every name of the package facade resolves (reference: tests/test_imports.py / test_public_api.py)."""
import metal_marlin_b200 as mm


def test_all_exports_resolve():
    missing = []
    for name in mm.__all__:
        try:
            getattr(mm, name)
        except Exception as e:      # noqa: BLE001 - the test reports every failing name at once
            missing.append((name, repr(e)[:120]))
    assert not missing, missing
    assert issubclass(mm.MarlinPipeline, mm.MMFP4Pipeline) and mm.KVCacheTorch is mm.KVCache
    assert len(mm.__all__) > 150 and "TrellisForCausalLM" in dir(mm)
