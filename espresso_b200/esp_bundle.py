"""`.esp` bundle: manifest (a small TOML dialect), directory layout, SHA-256 content catalog, referenced artifacts,
backend / profile selection, and the step from an opened bundle to decode engines.

Follows the reference's bundle contract:

* manifest fields, validation rules, rendering and parsing — ``ESPManifest``
  (Sources/ESPBundle/ESPBundle.swift:157-448): flat ``key = "value"`` lines, the four sections
  ``[compression_policy] [optimization] [output_head] [draft]``, string arrays on one line;
* layout and integrity — ``ESPBundleLayout`` / ``ESPBundleArchive`` (:450-694): ``manifest.toml``, ten required top-level
  directories, ``signatures/content-hashes.json`` holding the manifest hash and one hash per regular file;
* selection — ``ESPRuntimeResolver.selectBackend`` (Sources/ESPRuntime/ESPRuntimeContracts.swift:74-137), with one more
  backend kind, ``"cuda"``, preferred when a CUDA device is present.

Host-side only.  Errors carry the reference's case name in ``kind``.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from dataclasses import dataclass, field
from typing import Optional

MODEL_FAMILIES = ("gpt2", "llama", "qwen")
BACKEND_KINDS = ("ane-private", "cpu-safe", "cuda")  # "cuda": this library (not in the reference's enum)
PROFILES = ("prefill_256", "prefill_2048", "decode_1", "decode_2")
MODEL_TIERS = ("compat", "optimized", "native_fast")
BEHAVIOR_CLASSES = ("exact", "near_exact", "approximate")
OUTPUT_HEAD_KINDS = ("dense", "factored")
DRAFT_KINDS = ("exact_two_token", "multi_token")

MANIFEST_FILE = "manifest.toml"
SIGNATURE_CATALOG = "content-hashes.json"
REQUIRED_TOP_LEVEL = ("arch", "tokenizer", "weights", "graphs", "states", "adapters", "compiled", "benchmarks", "licenses", "signatures")


class BundleError(ValueError):
    """``kind`` is the reference's ``ESPBundleValidationError`` / ``ESPRuntimeSelectionError`` case name."""

    def __init__(self, kind: str, detail: str = ""):
        super().__init__(f"{kind}({detail})" if detail else kind)
        self.kind = kind
        self.detail = detail


@dataclass
class CompressionPolicy:
    name: str
    weight_bits: int
    activation_bits: Optional[int] = None


@dataclass
class OptimizationMetadata:
    recipe: str = "legacy"
    quality_gate: str = "legacy-compatible"
    teacher_model: Optional[str] = None
    draft_model: Optional[str] = None
    performance_target: Optional[str] = None


@dataclass
class OutputHeadMetadata:
    kind: str
    behavior_class: str
    bottleneck: Optional[int] = None
    groups: Optional[int] = None
    projection_ref: Optional[str] = None
    expansion_ref: Optional[str] = None


@dataclass
class DraftMetadata:
    kind: str
    behavior_class: str
    horizon: int
    verifier: str
    rollback: str
    artifact_ref: str
    acceptance_metric: str


def _non_empty(value: Optional[str], name: str) -> None:
    if value is None or not value.strip():
        raise BundleError("emptyField", name)


@dataclass
class Manifest:
    format_version: str
    model_id: str
    model_family: str
    architecture_version: str
    tokenizer_contract: str
    supported_backends: list
    supported_profiles: list
    max_context: int
    compression_policy: CompressionPolicy
    adapter_slots: int
    accuracy_baseline_ref: str
    performance_baseline_ref: str
    signature_ref: str
    context_target_tokens: Optional[int] = None
    model_tier: str = "compat"
    behavior_class: str = "exact"
    optimization: OptimizationMetadata = field(default_factory=OptimizationMetadata)
    output_head: Optional[OutputHeadMetadata] = None
    draft: Optional[DraftMetadata] = None

    def __post_init__(self):
        if self.context_target_tokens is None:
            self.context_target_tokens = self.max_context

    # ---- validation (ESPBundle.swift:222-262, 396-447) ------------------------------------------------------
    def validate(self) -> None:
        for value, name in ((self.format_version, "format_version"), (self.model_id, "model_id"),
                            (self.architecture_version, "architecture_version"), (self.tokenizer_contract, "tokenizer_contract"),
                            (self.accuracy_baseline_ref, "accuracy_baseline_ref"), (self.performance_baseline_ref, "performance_baseline_ref"),
                            (self.signature_ref, "signature_ref")):
            _non_empty(value, name)
        if not self.supported_backends:
            raise BundleError("missingBackends")
        if not self.supported_profiles:
            raise BundleError("missingProfiles")
        if self.max_context <= 0:
            raise BundleError("invalidMaxContext", str(self.max_context))
        if not 0 < self.context_target_tokens <= self.max_context:
            raise BundleError("invalidContextTarget", str(self.context_target_tokens))
        if self.adapter_slots < 0:
            raise BundleError("invalidAdapterSlots", str(self.adapter_slots))
        if self.compression_policy.weight_bits <= 0:
            raise BundleError("invalidWeightBits", str(self.compression_policy.weight_bits))
        if self.compression_policy.activation_bits is not None and self.compression_policy.activation_bits <= 0:
            raise BundleError("invalidActivationBits", str(self.compression_policy.activation_bits))
        _non_empty(self.optimization.recipe, "optimization.recipe")
        _non_empty(self.optimization.quality_gate, "optimization.quality_gate")
        head = self.output_head
        if head is not None:
            if self.model_family != "llama":
                raise BundleError("invalidOutputHead", "output-head metadata is supported for llama bundles only")
            if head.kind == "dense":
                if any(v is not None for v in (head.bottleneck, head.groups, head.projection_ref, head.expansion_ref)):
                    raise BundleError("invalidOutputHead", "dense output head cannot declare factored weights or dimensions")
            else:
                if head.bottleneck is None or head.bottleneck <= 0:
                    raise BundleError("invalidOutputHead", "factored output head requires bottleneck > 0")
                if head.groups is None or head.groups <= 0:
                    raise BundleError("invalidOutputHead", "factored output head requires groups > 0")
                _non_empty(head.projection_ref, "output_head.projection_ref")
                _non_empty(head.expansion_ref, "output_head.expansion_ref")
        draft = self.draft
        if draft is not None:
            if self.model_family != "llama":
                raise BundleError("invalidDraft", "draft metadata is supported for llama bundles only")
            if draft.kind != "exact_two_token":
                raise BundleError("invalidDraft", "only exact_two_token drafts are currently supported")
            if draft.horizon <= 1:
                raise BundleError("invalidDraft", "draft horizon must be > 1")
            if draft.horizon != 2:
                raise BundleError("invalidDraft", "exact_two_token draft requires horizon == 2")
            _non_empty(draft.verifier, "draft.verifier")
            _non_empty(draft.rollback, "draft.rollback")
            _non_empty(draft.acceptance_metric, "draft.acceptance_metric")
            _non_empty(draft.artifact_ref, "draft.artifact_ref")

    # ---- TOML (ESPBundle.swift:264-394) ------------------------------------------------------------------------
    def render_toml(self) -> str:
        q = lambda v: f'"{v}"'  # noqa: E731
        qa = lambda vs: "[" + ", ".join(q(v) for v in vs) + "]"  # noqa: E731
        cp, op, head, draft = self.compression_policy, self.optimization, self.output_head, self.draft
        lines = [
            f"format_version = {q(self.format_version)}", f"model_id = {q(self.model_id)}", f"model_family = {q(self.model_family)}",
            f"architecture_version = {q(self.architecture_version)}", f"tokenizer_contract = {q(self.tokenizer_contract)}",
            f"supported_backends = {qa(self.supported_backends)}", f"supported_profiles = {qa(self.supported_profiles)}",
            f"max_context = {self.max_context}", f"context_target_tokens = {self.context_target_tokens}",
            f"model_tier = {q(self.model_tier)}", f"behavior_class = {q(self.behavior_class)}", f"adapter_slots = {self.adapter_slots}",
            f"accuracy_baseline_ref = {q(self.accuracy_baseline_ref)}", f"performance_baseline_ref = {q(self.performance_baseline_ref)}",
            f"signature_ref = {q(self.signature_ref)}",
            "[compression_policy]", f"name = {q(cp.name)}", f"weight_bits = {cp.weight_bits}",
            None if cp.activation_bits is None else f"activation_bits = {cp.activation_bits}",
            "[optimization]", f"recipe = {q(op.recipe)}", f"quality_gate = {q(op.quality_gate)}",
            None if op.teacher_model is None else f"teacher_model = {q(op.teacher_model)}",
            None if op.draft_model is None else f"draft_model = {q(op.draft_model)}",
            None if op.performance_target is None else f"performance_target = {q(op.performance_target)}",
        ]
        if head is not None:
            lines += ["[output_head]", f"kind = {q(head.kind)}", f"behavior_class = {q(head.behavior_class)}",
                      None if head.bottleneck is None else f"bottleneck = {head.bottleneck}",
                      None if head.groups is None else f"groups = {head.groups}",
                      None if head.projection_ref is None else f"projection_ref = {q(head.projection_ref)}",
                      None if head.expansion_ref is None else f"expansion_ref = {q(head.expansion_ref)}"]
        if draft is not None:
            lines += ["[draft]", f"kind = {q(draft.kind)}", f"behavior_class = {q(draft.behavior_class)}", f"horizon = {draft.horizon}",
                      f"verifier = {q(draft.verifier)}", f"rollback = {q(draft.rollback)}", f"artifact_ref = {q(draft.artifact_ref)}",
                      f"acceptance_metric = {q(draft.acceptance_metric)}"]
        return "\n".join(line for line in lines if line is not None) + "\n"

    @classmethod
    def parse_toml(cls, text: str) -> "Manifest":
        sections: dict[Optional[str], dict[str, str]] = {None: {}, "compression_policy": {}, "optimization": {}, "output_head": {}, "draft": {}}
        current: Optional[str] = None
        for raw in text.splitlines():
            line = raw.strip()
            if not line or line.startswith("#"):
                continue
            if line.startswith("["):
                name = line[1:-1] if line.endswith("]") else None
                if name not in ("compression_policy", "optimization", "output_head", "draft"):
                    raise BundleError("malformedSection", line)
                current = name
                continue
            if "=" not in line:
                raise BundleError("malformedLine", line)
            key, value = line.split("=", 1)
            sections[current][key.strip()] = value.strip()
        top, cp, op, oh, dr = (sections[k] for k in (None, "compression_policy", "optimization", "output_head", "draft"))

        def unquote(value: str) -> str:
            t = value.strip()
            if len(t) < 2 or not (t.startswith('"') and t.endswith('"')):
                raise BundleError("unsupportedValue", value)
            return t[1:-1]

        def string(d, key, default=None):
            if key not in d:
                if default is not None:
                    return default
                raise BundleError("emptyField", key)
            return unquote(d[key])

        def integer(d, key):
            try:
                return int(d[key])
            except (KeyError, ValueError):
                raise BundleError("unsupportedValue", key) from None

        def opt_int(d, key):
            try:
                return int(d[key])
            except (KeyError, ValueError):
                return None

        def opt_string(d, key):
            try:
                return unquote(d[key])
            except (KeyError, BundleError):
                return None

        def enum(d, key, allowed, default=None):
            if key not in d and default is not None:
                return default
            raw = string(d, key)
            if raw not in allowed:
                raise BundleError("unsupportedValue", raw)
            return raw

        def array(d, key, allowed):
            if key not in d:
                raise BundleError("emptyField", key)
            t = d[key].strip()
            if not (t.startswith("[") and t.endswith("]")):
                raise BundleError("unsupportedValue", d[key])
            body = t[1:-1]
            if not body.strip():
                return []
            out = []
            for part in body.split(","):
                v = unquote(part.strip())
                if v not in allowed:
                    raise BundleError("unsupportedValue", v)
                out.append(v)
            return out

        head = None
        if oh:
            head = OutputHeadMetadata(enum(oh, "kind", OUTPUT_HEAD_KINDS), enum(oh, "behavior_class", BEHAVIOR_CLASSES), opt_int(oh, "bottleneck"),
                                      opt_int(oh, "groups"), opt_string(oh, "projection_ref"), opt_string(oh, "expansion_ref"))
        draft = None
        if dr:
            draft = DraftMetadata(enum(dr, "kind", DRAFT_KINDS), enum(dr, "behavior_class", BEHAVIOR_CLASSES), integer(dr, "horizon"),
                                  string(dr, "verifier"), string(dr, "rollback"), string(dr, "artifact_ref"), string(dr, "acceptance_metric"))
        m = cls(
            format_version=string(top, "format_version"), model_id=string(top, "model_id"), model_family=enum(top, "model_family", MODEL_FAMILIES),
            architecture_version=string(top, "architecture_version"), tokenizer_contract=string(top, "tokenizer_contract"),
            supported_backends=array(top, "supported_backends", BACKEND_KINDS), supported_profiles=array(top, "supported_profiles", PROFILES),
            max_context=integer(top, "max_context"), context_target_tokens=opt_int(top, "context_target_tokens"),
            compression_policy=CompressionPolicy(string(cp, "name"), integer(cp, "weight_bits"), opt_int(cp, "activation_bits")),
            model_tier=enum(top, "model_tier", MODEL_TIERS, "compat"), behavior_class=enum(top, "behavior_class", BEHAVIOR_CLASSES, "exact"),
            adapter_slots=integer(top, "adapter_slots"),
            optimization=OptimizationMetadata(string(op, "recipe", "legacy"), string(op, "quality_gate", "legacy-compatible"),
                                              opt_string(op, "teacher_model"), opt_string(op, "draft_model"), opt_string(op, "performance_target")),
            output_head=head, draft=draft, accuracy_baseline_ref=string(top, "accuracy_baseline_ref"),
            performance_baseline_ref=string(top, "performance_baseline_ref"), signature_ref=string(top, "signature_ref"))
        m.validate()
        return m


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


@dataclass
class BundleArchive:
    bundle_dir: str
    manifest: Manifest

    @property
    def manifest_path(self) -> str:
        return os.path.join(self.bundle_dir, MANIFEST_FILE)

    @property
    def weights_dir(self) -> str:
        return os.path.join(self.bundle_dir, "weights")

    @property
    def tokenizer_dir(self) -> str:
        return os.path.join(self.bundle_dir, "tokenizer")

    @property
    def signature_catalog_path(self) -> str:
        return os.path.join(self.bundle_dir, "signatures", SIGNATURE_CATALOG)

    # ---- integrity (ESPBundle.swift:601-649) --------------------------------------------------------------------
    def compute_catalog(self) -> dict:
        root = os.path.realpath(self.bundle_dir)
        hashes = {}
        for base, _, files in os.walk(root):
            for name in files:
                full = os.path.join(base, name)
                if name == MANIFEST_FILE or os.path.realpath(full) == os.path.realpath(self.signature_catalog_path):
                    continue
                if os.path.isfile(full):
                    hashes[os.path.relpath(os.path.realpath(full), root).replace(os.sep, "/")] = _sha256(full)
        return {"algorithm": "sha256", "manifestHash": _sha256(self.manifest_path), "fileHashes": dict(sorted(hashes.items()))}

    def write_signature_catalog(self) -> None:
        with open(self.signature_catalog_path, "w", encoding="utf-8") as f:
            json.dump(self.compute_catalog(), f, indent=2, sort_keys=True)

    def verify_signatures(self) -> None:
        with open(self.signature_catalog_path, "r", encoding="utf-8") as f:
            catalog = json.load(f)
        computed = self.compute_catalog()
        if catalog.get("manifestHash") != computed["manifestHash"]:
            raise BundleError("signatureMismatch", MANIFEST_FILE)
        for path, expected in sorted((catalog.get("fileHashes") or {}).items()):
            if computed["fileHashes"].get(path) != expected:
                raise BundleError("signatureMismatch", path)

    # ---- referenced artifacts (ESPBundle.swift:651-693) ----------------------------------------------------------
    def resolve_reference(self, reference: str) -> str:
        if not reference or reference.startswith("/"):
            raise BundleError("invalidReferencedPath", reference)
        root = os.path.normpath(os.path.abspath(self.bundle_dir))
        resolved = os.path.normpath(os.path.join(root, reference))
        if resolved != root and not resolved.startswith(root + os.sep):
            raise BundleError("invalidReferencedPath", reference)
        return resolved

    def validate_referenced_artifacts(self) -> None:
        refs = []
        head = self.manifest.output_head
        if head is not None and head.kind == "factored":
            refs += [r for r in (head.projection_ref, head.expansion_ref) if r is not None]
        if self.manifest.draft is not None:
            refs.append(self.manifest.draft.artifact_ref)
        for ref in refs:
            if not os.path.isfile(self.resolve_reference(ref)):
                raise BundleError("missingReferencedFile", ref)

    # ---- create / open (ESPBundle.swift:541-599) -------------------------------------------------------------------
    @classmethod
    def create(cls, bundle_dir: str, manifest: Manifest, weights_directory: str, tokenizer_directory: str,
               overwrite_existing: bool = False) -> "BundleArchive":
        manifest.validate()
        if os.path.exists(bundle_dir):
            if not overwrite_existing:
                raise FileExistsError(bundle_dir)
            shutil.rmtree(bundle_dir)
        os.makedirs(bundle_dir)
        for entry in REQUIRED_TOP_LEVEL:
            os.makedirs(os.path.join(bundle_dir, entry), exist_ok=True)
        archive = cls(bundle_dir, manifest)
        with open(archive.manifest_path, "w", encoding="utf-8") as f:
            f.write(manifest.render_toml())
        shutil.copytree(weights_directory, archive.weights_dir, dirs_exist_ok=True)
        shutil.copytree(tokenizer_directory, archive.tokenizer_dir, dirs_exist_ok=True)
        archive.write_signature_catalog()
        return archive

    @classmethod
    def open(cls, bundle_dir: str, verify_signatures: bool = True) -> "BundleArchive":
        manifest_path = os.path.join(bundle_dir, MANIFEST_FILE)
        if not os.path.isfile(manifest_path):
            raise BundleError("missingManifest")
        for entry in REQUIRED_TOP_LEVEL:
            if not os.path.isdir(os.path.join(bundle_dir, entry)):
                raise BundleError("missingTopLevelEntry", entry)
        with open(manifest_path, "r", encoding="utf-8") as f:
            manifest = Manifest.parse_toml(f.read())
        archive = cls(bundle_dir, manifest)
        if verify_signatures:
            archive.verify_signatures()
        archive.validate_referenced_artifacts()
        return archive


# ---- runtime selection (ESPRuntimeContracts.swift:74-137) ------------------------------------------------------------

@dataclass
class DeviceCapabilities:
    supports_ane_private: bool = False
    supports_cuda: bool = False


@dataclass
class RuntimeSelection:
    backend: str
    profile: str
    context_target_tokens: int
    output_head: Optional[OutputHeadMetadata]
    draft: Optional[DraftMetadata]
    reason: str


def select_profile(manifest: Manifest) -> str:
    if manifest.context_target_tokens > 256:
        for p in ("prefill_2048", "prefill_256"):
            if p in manifest.supported_profiles:
                return p
    elif "prefill_256" in manifest.supported_profiles:
        return "prefill_256"
    if manifest.supported_profiles:
        return manifest.supported_profiles[0]
    raise BundleError("noCompatibleProfile")


def select_backend(capabilities: DeviceCapabilities, manifest: Manifest, requested_context_tokens: Optional[int] = None,
                   preferred=("cuda", "ane-private", "cpu-safe")) -> RuntimeSelection:
    manifest.validate()
    if requested_context_tokens is not None and requested_context_tokens > manifest.context_target_tokens:
        raise BundleError("requestedContextExceedsTarget", f"requested: {requested_context_tokens}, supported: {manifest.context_target_tokens}")
    profile = select_profile(manifest)
    for backend in preferred:
        if backend not in manifest.supported_backends:
            continue
        if backend == "cuda" and capabilities.supports_cuda:
            reason = "CUDA backend is available on this host"
        elif backend == "ane-private" and capabilities.supports_ane_private:
            reason = "Private ANE backend is available on this host"
        elif backend == "cpu-safe":
            reason = "Fell back to CPU-safe backend"
        else:
            continue
        return RuntimeSelection(backend, profile, manifest.context_target_tokens, manifest.output_head, manifest.draft, reason)
    raise BundleError("noCompatibleBackend")


def draft_environment(manifest: Manifest) -> dict:
    """The variables the bundled runtime hands to the engine for a ``[draft]`` section
    (Sources/ESPRuntime/ESPBundledRuntime.swift:169-177)."""
    d = manifest.draft
    if d is None:
        return {}
    return {
        "ESPRESSO_BUNDLE_DRAFT_KIND": d.kind, "ESPRESSO_BUNDLE_DRAFT_HORIZON": str(d.horizon),
        "ESPRESSO_BUNDLE_DRAFT_VERIFIER": d.verifier, "ESPRESSO_BUNDLE_DRAFT_ROLLBACK": d.rollback,
        "ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF": d.artifact_ref, "ESPRESSO_BUNDLE_DRAFT_ACCEPTANCE_METRIC": d.acceptance_metric,
    }


@dataclass
class ResolvedDraft:
    model_dir: str                 # the descriptor's model_dir as written
    tokenizer_dir: Optional[str]
    model_id: Optional[str]
    descriptor_path: str
    weight_dir: str                # absolute directory of the draft model's weights
    config: "object"               # its MultiModelConfig


def _inside(path: str, root: str) -> bool:
    return path == root or path.startswith(root + os.sep)


def resolve_exact_two_token_draft(config, weight_dir: str, environment) -> Optional[ResolvedDraft]:
    """Where the exact two-token draft of a model lives, or None when none is asked for
    (``resolveExactTwoTokenDraft``, Sources/RealModelInference/RealModelInferenceEngine.swift:5324-5390).

    ``ESPRESSO_BUNDLE_DRAFT_KIND`` must be ``exact_two_token``; a horizon, if given, must be 2;
    ``ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF`` names a JSON descriptor relative to the bundle root (the parent of the weight
    directory) and may not leave it; the descriptor's ``model_dir`` is relative to the weight directory and may not leave
    that; the draft must be a llama model with the target's vocabulary.  Failures raise ``BundleError("runtimeFailure")``
    with the reference's message."""
    from .model_config import MultiModelConfig

    def fail(msg: str):
        return BundleError("runtimeFailure", msg)

    if environment.get("ESPRESSO_BUNDLE_DRAFT_KIND") != "exact_two_token":
        return None
    raw_horizon = environment.get("ESPRESSO_BUNDLE_DRAFT_HORIZON")
    if raw_horizon is not None:
        try:
            horizon = int(raw_horizon)
        except ValueError:
            horizon = None
        if horizon != 2:
            raise fail(f"exact two-token draft requires horizon == 2, got {raw_horizon}")
    artifact_ref = environment.get("ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF")
    if not artifact_ref:
        raise fail("exact two-token draft requires ESPRESSO_BUNDLE_DRAFT_ARTIFACT_REF")
    weight_root = os.path.normpath(os.path.abspath(weight_dir))
    bundle_root = os.path.dirname(weight_root)
    descriptor_path = os.path.normpath(os.path.join(bundle_root, artifact_ref))
    if not _inside(descriptor_path, bundle_root):
        raise fail(f"Draft artifact ref escapes bundle root: {artifact_ref}")
    if not os.path.exists(descriptor_path):
        raise fail(f"Draft artifact file is missing: {descriptor_path}")
    try:
        with open(descriptor_path) as f:
            desc = json.load(f)
        model_dir = desc["model_dir"]
        if not isinstance(model_dir, str):
            raise TypeError("model_dir must be a string")
    except (OSError, ValueError, KeyError, TypeError) as e:
        raise fail(f"Failed to decode draft descriptor {descriptor_path}: {e}")
    if not model_dir:
        raise fail("Draft descriptor is missing model_dir")
    draft_dir = os.path.normpath(os.path.join(weight_root, model_dir))
    if not _inside(draft_dir, weight_root):
        raise fail(f"Draft model_dir escapes weights root: {model_dir}")
    if not os.path.isdir(draft_dir):
        raise fail(f"Weight directory does not exist: {draft_dir}")
    try:
        draft_config = MultiModelConfig.load(draft_dir)
    except (OSError, ValueError, KeyError) as e:
        raise fail(f"Failed to load draft metadata in {draft_dir}: {e}")
    if draft_config.architecture != "llama":
        raise fail("exact two-token draft currently supports llama draft models only")
    if draft_config.vocab != config.vocab:
        raise fail(f"draft/full vocab mismatch: draft={draft_config.vocab} full={config.vocab}")
    return ResolvedDraft(model_dir, desc.get("tokenizer_dir"), desc.get("model_id"), descriptor_path, draft_dir, draft_config)


def open_engines(archive: BundleArchive, max_batch: int = 1, device: int = 0, flags: int = 0):
    """``(target engine, draft engine or None, tokenizer)`` for a bundle whose selection is the ``cuda`` backend: the
    weights directory feeds the engine; a ``[draft]`` section becomes the variables of ``draft_environment`` and the
    draft's weight directory is resolved from them as the reference does (``resolve_exact_two_token_draft``); the
    tokenizer files are searched in ``tokenizer/``."""
    from . import runtime, tokenizers
    from .model_config import MultiModelConfig

    cfg = MultiModelConfig.load(archive.weights_dir)
    resolved = resolve_exact_two_token_draft(cfg, archive.weights_dir, draft_environment(archive.manifest))
    target = runtime.DecodeEngine.build(archive.weights_dir, max_batch=max_batch, device=device, flags=flags)
    draft = None
    if resolved is not None:
        draft = runtime.DecodeEngine.build(resolved.weight_dir, max_batch=1, device=device, flags=flags)
    try:
        tokenizer = tokenizers.load_tokenizer(cfg.architecture, archive.tokenizer_dir)
    except FileNotFoundError:
        tokenizer = None
    return target, draft, tokenizer
