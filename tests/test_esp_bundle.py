"""`.esp` bundle contract: the reference's manifest tests (Tests/ESPBundleTests/ESPManifestTests.swift) restated, plus
create / open / tamper detection and backend selection with the added `cuda` kind."""
import dataclasses
import json
import os

import pytest

from espresso_b200 import esp_bundle as eb


def full_manifest(**over):
    kw = dict(
        format_version="1.1.0", model_id="espresso.llama.1b", model_family="llama", architecture_version="decoder-v1",
        tokenizer_contract="sentencepiece-v1", supported_backends=["ane-private", "cpu-safe"],
        supported_profiles=["prefill_256", "prefill_2048", "decode_1"], max_context=2048, context_target_tokens=1024,
        compression_policy=eb.CompressionPolicy("int4-palettized", 4, None), model_tier="optimized", behavior_class="near_exact",
        adapter_slots=4,
        optimization=eb.OptimizationMetadata("stories-gqa4-distilled", "short-long-prompt-parity", "teacher://qwen3-0.6b", None, "110 tok/s"),
        output_head=eb.OutputHeadMetadata("factored", "near_exact", 128, 1, "weights/cls_proj.bin", "weights/cls_expand.bin"),
        draft=eb.DraftMetadata("exact_two_token", "exact", 2, "exact", "exact_replay", "weights/future-sidecar.bin", "accepted_future_tokens"),
        accuracy_baseline_ref="benchmarks/qwen-0.6b/accuracy.json", performance_baseline_ref="benchmarks/qwen-0.6b/perf.json",
        signature_ref="signatures/manifest.sig")
    kw.update(over)
    return eb.Manifest(**kw)


def test_manifest_rendering_is_deterministic_and_round_trips():
    m = full_manifest()
    a = m.render_toml()
    assert a == m.render_toml()
    for needle in ('model_family = "llama"', 'model_tier = "optimized"', 'behavior_class = "near_exact"', "context_target_tokens = 1024",
                   'supported_backends = ["ane-private", "cpu-safe"]', "[output_head]", 'projection_ref = "weights/cls_proj.bin"', "[draft]",
                   'artifact_ref = "weights/future-sidecar.bin"'):
        assert needle in a
    assert eb.Manifest.parse_toml(a) == m


def test_parser_backfills_defaults_for_legacy_bundles():
    text = '''
    format_version = "1.0.0"
    model_id = "legacy.stories"
    model_family = "llama"
    architecture_version = "decoder-v1"
    tokenizer_contract = "sentencepiece-v1"
    supported_backends = ["ane-private", "cpu-safe"]
    supported_profiles = ["prefill_256", "decode_1"]
    max_context = 256
    adapter_slots = 0
    accuracy_baseline_ref = "benchmarks/accuracy.json"
    performance_baseline_ref = "benchmarks/perf.json"
    signature_ref = "signatures/content-hashes.json"
    [compression_policy]
    name = "native-ane-fp16"
    weight_bits = 16
    '''
    m = eb.Manifest.parse_toml(text)
    assert (m.model_tier, m.behavior_class, m.context_target_tokens) == ("compat", "exact", 256)
    assert (m.optimization.recipe, m.optimization.quality_gate) == ("legacy", "legacy-compatible")
    assert m.output_head is None and m.draft is None


@pytest.mark.parametrize("over,kind", [
    (dict(model_id="  "), "emptyField"),
    (dict(supported_backends=[]), "missingBackends"),
    (dict(supported_profiles=[]), "missingProfiles"),
    (dict(max_context=0), "invalidMaxContext"),
    (dict(context_target_tokens=4096), "invalidContextTarget"),
    (dict(adapter_slots=-1), "invalidAdapterSlots"),
    (dict(compression_policy=eb.CompressionPolicy("x", 0)), "invalidWeightBits"),
    (dict(compression_policy=eb.CompressionPolicy("x", 4, 0)), "invalidActivationBits"),
    (dict(model_family="gpt2"), "invalidOutputHead"),
    (dict(model_family="qwen", output_head=None), "invalidDraft"),
    (dict(output_head=eb.OutputHeadMetadata("factored", "exact", None, 1, "a", "b")), "invalidOutputHead"),
    (dict(output_head=eb.OutputHeadMetadata("dense", "exact", 8)), "invalidOutputHead"),
    (dict(draft=eb.DraftMetadata("multi_token", "exact", 2, "v", "r", "a", "m")), "invalidDraft"),
    (dict(draft=eb.DraftMetadata("exact_two_token", "exact", 3, "v", "r", "a", "m")), "invalidDraft"),
    (dict(draft=eb.DraftMetadata("exact_two_token", "exact", 2, "v", "r", "", "m")), "emptyField"),
])
def test_validation_rejects(over, kind):
    with pytest.raises(eb.BundleError) as e:
        full_manifest(**over).validate()
    assert e.value.kind == kind


def test_parser_error_kinds():
    good = full_manifest().render_toml()
    for text, kind in ((good.replace("[draft]", "[drafts]"), "malformedSection"), (good + "\nno equals sign\n", "malformedLine"),
                       (good.replace('model_family = "llama"', 'model_family = "bert"'), "unsupportedValue"),
                       (good.replace("max_context = 2048", "max_context = lots"), "unsupportedValue"),
                       (good.replace('model_id = "espresso.llama.1b"\n', ""), "emptyField")):
        with pytest.raises(eb.BundleError) as e:
            eb.Manifest.parse_toml(text)
        assert e.value.kind == kind, text[:60]


def make_dirs(tmp_path):
    w, t = tmp_path / "w", tmp_path / "t"
    (w / "layers" / "0").mkdir(parents=True)
    t.mkdir()
    (w / "lm_head.bin").write_bytes(b"\x01" * 64)
    (w / "layers" / "0" / "wq.bin").write_bytes(b"\x02" * 64)
    (w / "cls_proj.bin").write_bytes(b"p")
    (w / "cls_expand.bin").write_bytes(b"e")
    (w / "future-sidecar.bin").write_bytes(b"d")
    (t / "tokenizer.json").write_text("{}")
    return str(w), str(t)


def test_bundle_create_open_round_trip_and_tamper_detection(tmp_path):
    w, t = make_dirs(tmp_path)
    bundle = str(tmp_path / "model.esp")
    created = eb.BundleArchive.create(bundle, full_manifest(), w, t)
    for entry in eb.REQUIRED_TOP_LEVEL:
        assert os.path.isdir(os.path.join(bundle, entry))
    catalog = json.load(open(created.signature_catalog_path))
    assert catalog["algorithm"] == "sha256" and "weights/layers/0/wq.bin" in catalog["fileHashes"] and "manifest.toml" not in catalog["fileHashes"]
    opened = eb.BundleArchive.open(bundle)
    assert opened.manifest == created.manifest
    with pytest.raises(FileExistsError):
        eb.BundleArchive.create(bundle, full_manifest(), w, t)
    open(os.path.join(bundle, "weights", "lm_head.bin"), "wb").write(b"\x09" * 64)
    with pytest.raises(eb.BundleError) as e:
        eb.BundleArchive.open(bundle)
    assert e.value.kind == "signatureMismatch" and e.value.detail == "weights/lm_head.bin"
    eb.BundleArchive.open(bundle, verify_signatures=False)  # content checks are optional, as in the reference
    os.rmdir(os.path.join(bundle, "graphs"))
    with pytest.raises(eb.BundleError) as e:
        eb.BundleArchive.open(bundle, verify_signatures=False)
    assert e.value.kind == "missingTopLevelEntry" and e.value.detail == "graphs"
    with pytest.raises(eb.BundleError) as e:
        eb.BundleArchive.open(str(tmp_path / "nothing.esp"))
    assert e.value.kind == "missingManifest"


def test_bundle_open_rejects_missing_or_escaping_references(tmp_path):
    w, t = make_dirs(tmp_path)
    os.remove(os.path.join(w, "future-sidecar.bin"))
    bundle = str(tmp_path / "model.esp")
    eb.BundleArchive.create(bundle, full_manifest(), w, t)
    with pytest.raises(eb.BundleError) as e:
        eb.BundleArchive.open(bundle)
    assert e.value.kind == "missingReferencedFile" and e.value.detail == "weights/future-sidecar.bin"
    archive = eb.BundleArchive(bundle, full_manifest())
    for bad in ("/etc/passwd", "../outside.bin", ""):
        with pytest.raises(eb.BundleError) as e:
            archive.resolve_reference(bad)
        assert e.value.kind == "invalidReferencedPath"


def test_backend_and_profile_selection():
    m = full_manifest(supported_backends=["ane-private", "cpu-safe", "cuda"])
    sel = eb.select_backend(eb.DeviceCapabilities(supports_cuda=True), m)
    assert (sel.backend, sel.profile, sel.context_target_tokens) == ("cuda", "prefill_2048", 1024) and sel.draft == m.draft
    assert eb.select_backend(eb.DeviceCapabilities(), m).backend == "cpu-safe"
    assert eb.select_backend(eb.DeviceCapabilities(supports_ane_private=True), m).backend == "ane-private"
    assert eb.select_backend(eb.DeviceCapabilities(supports_cuda=True), full_manifest()).backend == "cpu-safe"  # bundle without the cuda kind
    with pytest.raises(eb.BundleError) as e:
        eb.select_backend(eb.DeviceCapabilities(), full_manifest(supported_backends=["ane-private"]))
    assert e.value.kind == "noCompatibleBackend"
    with pytest.raises(eb.BundleError) as e:
        eb.select_backend(eb.DeviceCapabilities(), m, requested_context_tokens=2000)
    assert e.value.kind == "requestedContextExceedsTarget"
    assert eb.select_profile(full_manifest(context_target_tokens=256, supported_profiles=["decode_1", "prefill_256"])) == "prefill_256"
    assert eb.select_profile(full_manifest(context_target_tokens=256, supported_profiles=["decode_2"])) == "decode_2"


def test_draft_descriptor_resolution_follows_the_reference(tmp_path):
    """The layout of the reference's own test (RealModelInferenceTests.swift:252-311): the artifact ref is relative to the
    bundle root, the descriptor's model_dir to the weight directory; then every way the resolution can fail."""
    from espresso_b200.model_config import MultiModelConfig

    cfg = MultiModelConfig("stories110m", 12, 12, 12, 768, 64, 2048, 32000, 256, 1e-5, 10000.0, None, "llama")
    weights = tmp_path / "bundle" / "weights"
    student = weights / "draft" / "student"
    student.mkdir(parents=True)
    dataclasses.replace(cfg, name="stories110m-stable-copy").save(str(student))
    desc = weights / "draft" / "exact-two-token.json"
    desc.write_text(json.dumps({"model_dir": "draft/student", "tokenizer_dir": "tokenizer", "model_id": "stories110m-stable-copy"}))
    env = {"ESPRESSO_BUNDLE_DRAFT_KIND": "exact_two_token", "ESPRESSO_BUNDLE_DRAFT_HORIZON": "2",
           "ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF": "weights/draft/exact-two-token.json"}
    r = eb.resolve_exact_two_token_draft(cfg, str(weights), env)
    assert r.weight_dir == str(student) and r.model_id == "stories110m-stable-copy" and r.config.nLayer == 12
    assert r.descriptor_path == str(desc) and r.tokenizer_dir == "tokenizer"
    # no draft asked for
    assert eb.resolve_exact_two_token_draft(cfg, str(weights), {}) is None
    assert eb.resolve_exact_two_token_draft(cfg, str(weights), dict(env, ESPRESSO_BUNDLE_DRAFT_KIND="multi_token")) is None
    # the horizon is optional, but if present it is 2
    assert eb.resolve_exact_two_token_draft(cfg, str(weights), {k: v for k, v in env.items() if "HORIZON" not in k}) is not None

    def fails(environment, config=cfg, text=""):
        with pytest.raises(eb.BundleError) as e:
            eb.resolve_exact_two_token_draft(config, str(weights), environment)
        assert e.value.kind == "runtimeFailure" and text in e.value.detail

    fails(dict(env, ESPRESSO_BUNDLE_DRAFT_HORIZON="3"), text="horizon == 2, got 3")
    fails(dict(env, ESPRESSO_BUNDLE_DRAFT_HORIZON="two"), text="horizon == 2")
    fails({k: v for k, v in env.items() if "ARTIFACT" not in k}, text="requires ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF")
    fails(dict(env, ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF=""), text="requires ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF")
    fails(dict(env, ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF="../elsewhere.json"), text="escapes bundle root")
    fails(dict(env, ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF="weights/draft/none.json"), text="is missing")
    fails(env, config=dataclasses.replace(cfg, vocab=32001), text="draft=32000 full=32001")
    desc.write_text("{not json")
    fails(env, text="Failed to decode draft descriptor")
    desc.write_text(json.dumps({"tokenizer_dir": "tokenizer"}))
    fails(env, text="Failed to decode draft descriptor")
    desc.write_text(json.dumps({"model_dir": ""}))
    fails(env, text="missing model_dir")
    desc.write_text(json.dumps({"model_dir": "../outside"}))
    fails(env, text="escapes weights root")
    desc.write_text(json.dumps({"model_dir": "draft/absent"}))
    fails(env, text="does not exist")
    desc.write_text(json.dumps({"model_dir": "draft/student"}))
    dataclasses.replace(cfg, architecture="gpt2").save(str(student))
    fails(env, text="llama draft models only")


def test_draft_environment_of_a_manifest():
    d = eb.DraftMetadata("exact_two_token", "exact", 2, "exact", "exact_replay", "weights/draft/exact-two-token.json", "accepted_future_tokens")
    env = eb.draft_environment(full_manifest(draft=d))
    assert env["ESPRESSO_BUNDLE_DRAFT_KIND"] == "exact_two_token" and env["ESPRESSO_BUNDLE_DRAFT_HORIZON"] == "2"
    assert env["ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF"] == "weights/draft/exact-two-token.json"
    assert env["ESPRESSO_BUNDLE_DRAFT_ROLLBACK"] == "exact_replay" and env["ESPRESSO_BUNDLE_DRAFT_ACCEPTANCE_METRIC"] == "accepted_future_tokens"
    assert eb.draft_environment(full_manifest(draft=None)) == {}


@pytest.mark.gpu
def test_bundle_to_engines_with_two_token_draft(tmp_path, tmp_models):
    """A bundle with a [draft] section opens into a target and a draft engine; the exact two-token loop matches greedy."""
    import shutil

    from espresso_b200.model_config import tiny_llama
    from espresso_b200.synthetic import synthetic_prompt

    cfg, dcfg = tiny_llama(vocab=96, max_seq=48, n_layer=2), tiny_llama(vocab=96, max_seq=48, n_layer=1)
    w = str(tmp_path / "weights_src")
    shutil.copytree(tmp_models(cfg), w)
    shutil.copytree(tmp_models(dcfg, 1235), os.path.join(w, "draft", "student"))
    with open(os.path.join(w, "draft", "exact-two-token.json"), "w") as f:
        json.dump({"model_dir": "draft/student", "tokenizer_dir": "tokenizer", "model_id": "student"}, f)
    t = tmp_path / "tok"
    t.mkdir()
    m = full_manifest(supported_backends=["cuda", "cpu-safe"], output_head=None, max_context=48, context_target_tokens=48,
                      draft=eb.DraftMetadata("exact_two_token", "exact", 2, "exact", "exact_replay", "weights/draft/exact-two-token.json", "accepted_future_tokens"))
    archive = eb.BundleArchive.open(eb.BundleArchive.create(str(tmp_path / "m.esp"), m, w, str(t)).bundle_dir)
    assert eb.select_backend(eb.DeviceCapabilities(supports_cuda=True), archive.manifest).backend == "cuda"
    target, draft, tokenizer = eb.open_engines(archive)
    assert draft is not None and tokenizer is None
    prompt = synthetic_prompt(cfg.vocab, 6)
    greedy = target.generate(prompt, 20).tokens
    two = target.generate_two_token(draft, prompt, 20)
    assert list(two.tokens) == list(greedy)
    draft.close()
    target.close()
