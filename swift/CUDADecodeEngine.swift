// Swift owner of a CUDA decode engine: the place CPUExactLlamaRuntime holds in
// Sources/RealModelInference/RealModelInferenceEngine.swift:548-850 and the first conformer of ESPRuntimeSession
// (Sources/ESPRuntime/ESPRuntimeContracts.swift:5-13).  Ownership and error conventions follow ANEKernel
// (Sources/ANERuntime/ANEKernel.swift:65-72, 440-444, 742-744): the handle is released in deinit, every failing call
// throws, nothing traps.
//
// Build: a system-library target over include/ (module.modulemap + espresso_cuda.h) named CEspressoCUDA, and this file
// in a target that depends on it and on ModelSupport / ANETypes / ESPRuntime.  No Swift toolchain exists on the
// machines this library is developed on, so this source has not been compiled there; every call below is exercised
// through the same C ABI by espresso_b200/runtime.py in the GPU test suite.

import CEspressoCUDA
import ModelSupport
import ANETypes

public enum CUDADecodeError: Error {
    case invalidArgument(String)      // ESP_CUDA_ERR_INVALID_ARGUMENT -> RealModelInferenceError.invalidGenerationParameters
    case outOfRange(String)           // position >= maxSeq or token >= vocab
    case io(String)                   // weight directory / file problems -> weightDirectoryNotFound / missingPath
    case timeout(String)              // a bounded device-side wait gave up
    case runtimeFailure(Int32, String)
}

public final class CUDADecodeEngine {
    private let handle: OpaquePointer
    public let config: MultiModelConfig

    public init(config: MultiModelConfig, weightDir: String, maxBatch: Int32 = 1, device: Int32 = 0, flags: UInt32 = 0) throws {
        var c = esp_cuda_config()
        c.architecture = config.architecture == .gpt2 ? 1 : 0
        c.n_layer = Int32(config.nLayer); c.n_head = Int32(config.nHead); c.n_kv_head = Int32(config.nKVHead)
        c.d_model = Int32(config.dModel); c.head_dim = Int32(config.headDim); c.hidden_dim = Int32(config.hiddenDim)
        c.vocab = Int32(config.vocab); c.max_seq = Int32(config.maxSeq); c.norm_eps = config.normEps
        c.rope_theta = config.ropeTheta; c.eos_token = config.eosToken.map { Int32($0) } ?? -1
        c.max_batch = maxBatch; c.device = device; c.tp_rank = 0; c.tp_size = 1; c.flags = flags
        var out: OpaquePointer?
        try Self.check(esp_cuda_create(&c, weightDir, &out))
        self.handle = out!
        self.config = config
    }

    /// GGUF files are parsed by the library; Q8_0 / Q4_0 blocks are uploaded as they are
    /// (replaces GGUFModelLoader.prepare, Sources/EspressoGGUF/GGUFModelLoader.swift:273-405).
    public init(ggufPath: String, config: MultiModelConfig, maxBatch: Int32 = 1, device: Int32 = 0, flags: UInt32 = 0) throws {
        var out: OpaquePointer?
        try Self.check(esp_cuda_create_from_gguf(ggufPath, maxBatch, device, flags, &out))
        self.handle = out!
        self.config = config
    }

    deinit { _ = esp_cuda_destroy(handle) }   // ANEKernel.deinit -> ane_interop_free

    // MARK: CPUExactLlamaRuntime surface (Engine.swift:613-670)
    public func reset() throws { try Self.check(esp_cuda_reset(handle)) }
    public func prefill(promptTokens: [TokenID]) throws {
        try Self.check(promptTokens.withUnsafeBufferPointer { esp_cuda_prefill(handle, $0.baseAddress, Int32($0.count)) })
    }
    public func advance(token: TokenID) throws { try Self.check(esp_cuda_advance(handle, token)) }
    public func selectGreedyToken() throws -> TokenID {
        var t: UInt32 = 0
        try Self.check(esp_cuda_select_greedy(handle, &t))
        return t
    }
    public func captureCheckpoint() throws -> Int32 {
        var id: Int32 = 0
        try Self.check(esp_cuda_checkpoint(handle, &id))
        return id
    }
    public func rollback(to id: Int32) throws { try Self.check(esp_cuda_rollback(handle, id)) }

    // MARK: ESPRuntimeSession (ESPRuntimeContracts.swift:5-13)
    public func decodeOne(_ token: TokenID) throws -> TokenID {
        var n: UInt32 = 0
        try Self.check(esp_cuda_decode_step(handle, token, &n))
        return n
    }
    public func decode(count: Int) throws -> [TokenID] {
        var out = [UInt32](repeating: 0, count: max(count, 1))
        var n: Int32 = 0
        try Self.check(esp_cuda_decode(handle, 1, Int32(count), &out, &n, nil))
        return Array(out.prefix(Int(n)))
    }
    /// Adapters (LoRA) are an ANE-graph feature of the reference (Sources/LoRAAdapter); this engine holds plain weights.
    public func attachAdapter(_ name: String) throws { throw CUDADecodeError.invalidArgument("adapters are not supported by the CUDA decode engine") }
    public func detachAdapter() throws {}
    /// Numeric fields the reference reports per session: kernel launches and device-time buckets of the last step.
    public func metrics() throws -> [String: Double] {
        var t = esp_cuda_timings()
        try Self.check(esp_cuda_get_timings(handle, &t))
        return ["qkv_ms": Double(t.qkv_ms), "attention_ms": Double(t.attention_ms), "ffn_ms": Double(t.ffn_ms),
                "head_ms": Double(t.head_ms), "total_ms": Double(t.total_ms), "kernel_launches": Double(t.kernel_launches)]
    }

    // MARK: generation (generate*ForTesting: token ids in, token ids out; Engine.swift:1405-1679)
    public struct Result {
        public var tokens: [TokenID]
        public var tokenLatenciesMs: [Double]
        public var tokensPerSecond: Double
        public var firstTokenLatencyMs: Double
        public var prefillMs: Double
        public var stoppedOnEOS: Bool
    }

    /// With `onStep` the loop runs token by token and the callback is invoked inline after every token
    /// (Engine.swift:6393-6405); without it the whole loop is driven on the device.
    public func generate(promptTokens: [TokenID], maxTokens: Int, onStep: ((TokenID, Int, Double) -> Void)? = nil) throws -> Result {
        var out = [UInt32](repeating: 0, count: max(maxTokens, 1))
        var n: Int32 = 0
        var res = esp_cuda_generation_result()
        if let onStep {
            let box = Unmanaged.passRetained(StepBox(onStep))
            defer { box.release() }
            try Self.check(promptTokens.withUnsafeBufferPointer {
                esp_cuda_generate_steps(handle, $0.baseAddress, Int32($0.count), Int32(maxTokens), { user, token, index, latency in
                    Unmanaged<StepBox>.fromOpaque(user!).takeUnretainedValue().call(token, Int(index), latency)
                }, box.toOpaque(), &out, &n, &res)
            })
        } else {
            try Self.check(promptTokens.withUnsafeBufferPointer {
                esp_cuda_generate(handle, $0.baseAddress, Int32($0.count), Int32(maxTokens), &out, &n, &res)
            })
        }
        var lat = [Float](repeating: 0, count: Int(config.maxSeq) + 1)
        var nl: Int32 = 0
        try Self.check(esp_cuda_token_latencies(handle, &lat, Int32(lat.count), &nl))
        return Result(tokens: Array(out.prefix(Int(n))), tokenLatenciesMs: lat.prefix(Int(nl)).map(Double.init),
                      tokensPerSecond: res.tokens_per_second, firstTokenLatencyMs: res.first_token_latency_ms,
                      prefillMs: res.prefill_ms, stoppedOnEOS: res.stopped_on_eos != 0)
    }

    // MARK: TwoTokenBranchVerifyingLanguageModel (Sources/Espresso/GenerationHarness.swift:239-252, 1281-1344)
    public func verifyPair(current: TokenID, proposedFuture: TokenID) throws -> (exactNext: TokenID, exactFuture: TokenID) {
        var a: UInt32 = 0, b: UInt32 = 0
        try Self.check(esp_cuda_verify2(handle, current, proposedFuture, &a, &b))
        return (a, b)
    }
    public func promote(stepCount: Int) throws { try Self.check(esp_cuda_commit(handle, Int32(stepCount))) }

    private final class StepBox {
        let call: (TokenID, Int, Double) -> Void
        init(_ f: @escaping (TokenID, Int, Double) -> Void) { call = f }
    }

    private static func check(_ status: Int32) throws {
        guard status != 0 else { return }
        let message = String(cString: esp_cuda_last_error_string())
        switch status {
        case 1: throw CUDADecodeError.invalidArgument(message)
        case 2: throw CUDADecodeError.outOfRange(message)
        case 5: throw CUDADecodeError.timeout(message)
        case 7: throw CUDADecodeError.io(message)
        default: throw CUDADecodeError.runtimeFailure(status, message)
        }
    }
}
