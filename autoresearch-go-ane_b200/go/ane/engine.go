// Package ane is the Go face of libane_b200.so: the same exported surface as the reference's
// ane package (ane/engine.go: Options, State, StepResult, Open, Step, EvalLogits, Flush, LR, SetLR,
// State, LoadState, Close, Prepare, SetGradTaskConcurrency) with every computation done by the
// CUDA library.  The binding is CGo-free: symbols are resolved with purego, like the reference's
// own Accelerate binding (ane/accel_darwin.go:74-82).
//
// This file cannot be compiled in the build container (no Go toolchain); it is kept
// deliberately plain: fixed-layout structs, integer and pointer arguments only, no callbacks,
// no Go pointer retained by C after a call returns.
//
// The stories package of the reference (model files, checkpoints, RandomInit) stays as it is and is
// imported here: Open reads Options.ModelPath with stories.LoadPretrained / stories.LoadCheckpoint and
// hands every tensor to the device with ImportTensor; SaveCheckpoint / LoadCheckpoint (checkpoint.go)
// go through stories.SaveCheckpoint / stories.LoadCheckpoint and the engine's own "SANE" trailer.
package ane

import (
	"fmt"
	"math/rand"
	"os"
	"runtime"
	"sync"
	"time"
	"unsafe"

	"github.com/ebitengine/purego"

	"github.com/tmc/autoresearch-go-ane/ane/stories"
)

// Options mirrors ane.Options of the reference (ane/engine.go:14-40) and adds the runtime model
// dimensions; zero values mean the reference defaults.
type Options struct {
	ModelPath         string
	Tokens            []uint16
	Seq               int
	AccumSteps        int
	LR                float32
	Seed              int64
	AdamBeta1         float32
	AdamBeta2         float32
	AdamEps           float32
	WeightDecay       float32
	GradClip          float32
	LossScale         float32
	CPUClassifierHead bool // accepted, ignored
	GradTaskLimit     int  // accepted, ignored
	UseANE            bool // accepted, ignored: the GPU path is always on
	HybridBackward    bool // accepted, ignored

	EmbedLRMult  float32
	ScalarLRMult float32
	LambdaLRMult float32
	LambdaBeta1  float32
	LambdaBeta2  float32

	// Additive fields.
	Dim, Hidden, Layers, Heads, KVHeads, Vocab int
	Batch                                      int
	Arch                                       int // 0 reference architecture, 1 llama-style
	ExactGradients                             bool
	FP32                                       bool
	Device, Rank, WorldSize                    int
	DPID                                       []byte // 128-byte bootstrap id when WorldSize > 1
	// NoModel lets a host that imports every tensor itself (ImportTensor) open an engine without a model
	// file; the reference has no such mode and rejects an empty ModelPath, which stays the default here.
	NoModel bool
}

// State mirrors ane.State (ane/engine.go:43-52).
type State struct {
	TokenPos     uint64
	LastLoss     float32
	CumTrainMS   float64
	CumWallMS    float64
	CumSteps     uint32
	CumBatches   uint32
	AdamT        uint32
	PendingSteps uint32
}

// StepResult mirrors ane.StepResult (ane/engine.go:55-69).
type StepResult struct {
	Loss                   float32
	StepDuration           time.Duration
	CompileDuration        time.Duration
	StartupCompileDuration time.Duration
	ANEEvalDuration        time.Duration // device time of the step
	CPUWorkDuration        time.Duration
	WeightRefreshDuration  time.Duration
	FinalHeadDuration      time.Duration
	EmbedGradDuration      time.Duration
	RMSDWDuration          time.Duration
	DWGEMMDuration         time.Duration
	DWWaitDuration         time.Duration
	AdamDuration           time.Duration
}

// C-side structs (include/ane_b200.h).  Field order and padding match the C layout.
type cOptions struct {
	structSize                                       uint32
	dim, hidden, nLayers, nHeads, nKVHeads, vocab    int32
	seq, batch, arch, quirks, computeDtype           int32
	ropeTheta                                        float32
	accumSteps                                       int32
	lr                                               float32
	seed                                             int64
	beta1, beta2, eps, weightDecay, gradClip, lossSc float32
	embedLRMult, scalarLRMult, lambdaLRMult          float32
	lambdaBeta1, lambdaBeta2                         float32
	useANE, hybridBackward, device, rank, worldSize  int32
	debugTaps, ceChunkRows, ceChunkCols              int32
	reserved                                         [5]int32
}

type cStepResult struct {
	structSize                                               uint32
	loss                                                     float32
	stepNS, compileNS, startupCompileNS, deviceEvalNS        int64
	cpuWorkNS, weightRefreshNS, finalHeadNS, embedGradNS     int64
	rmsDWNS, dwGEMMNS, dwWaitNS, adamNS                      int64
	flushed, deviceStatus                                    int32
}

type cState struct {
	structSize                                uint32
	cumSteps, cumBatches, adamT, pendingSteps uint32
	tokenPos                                  uint64
	lastLoss, pad                             float32
	cumTrainMS, cumWallMS                     float64
}

var (
	loadOnce sync.Once
	loadErr  error

	cOpen       func(opts *cOptions, tokens *uint16, nTokens uint64, dpID *byte, out *uintptr) int32
	cClose      func(e uintptr) int32
	cLastError  func(e uintptr) *byte
	cStep       func(e uintptr, out *cStepResult) int32
	cFlush      func(e uintptr, refreshMS *float64) int32
	cEvalLogits func(e uintptr, tokens *uint16, nSeq uint32, out *float32, outCap uint64, layout uint32) int32
	cHostMalloc func(bytes uint64) unsafe.Pointer
	cHostFree   func(p unsafe.Pointer) int32
	cEvalLoss   func(e uintptr, tokens *uint16, nSeq uint32, lossSum *float64, nPos *uint64) int32
	cSetLR      func(e uintptr, lr float32) int32
	cGetLR      func(e uintptr) float32
	cGetState   func(e uintptr, out *cState) int32
	cSetState   func(e uintptr, in *cState) int32
	cImport     func(e uintptr, id, layer, which uint32, buf *float32, n uint64) int32
	cExport     func(e uintptr, id, layer, which uint32, buf *float32, n uint64) int32
	cTensorSize func(e uintptr, id, layer uint32) int64
	cDecode     func(e uintptr, prompts *uint16, nSeq, promptLen, nNew uint32, temperature float32, uniforms *float64, out *uint16) int32
	cReseed     func(e uintptr, seed int64) int32
)

func load() error {
	loadOnce.Do(func() {
		path := os.Getenv("ANE_B200_LIB")
		if path == "" {
			path = "libane_b200.so"
		}
		lib, err := purego.Dlopen(path, purego.RTLD_NOW|purego.RTLD_GLOBAL)
		if err != nil {
			loadErr = fmt.Errorf("storiesane open: load %s: %w", path, err)
			return
		}
		purego.RegisterLibFunc(&cOpen, lib, "ane_open")
		purego.RegisterLibFunc(&cClose, lib, "ane_close")
		purego.RegisterLibFunc(&cLastError, lib, "ane_last_error")
		purego.RegisterLibFunc(&cStep, lib, "ane_step")
		purego.RegisterLibFunc(&cFlush, lib, "ane_flush")
		purego.RegisterLibFunc(&cEvalLogits, lib, "ane_eval_logits")
		purego.RegisterLibFunc(&cHostMalloc, lib, "ane_host_malloc")
		purego.RegisterLibFunc(&cHostFree, lib, "ane_host_free")
		purego.RegisterLibFunc(&cEvalLoss, lib, "ane_eval_loss")
		purego.RegisterLibFunc(&cSetLR, lib, "ane_set_lr")
		purego.RegisterLibFunc(&cGetLR, lib, "ane_get_lr")
		purego.RegisterLibFunc(&cGetState, lib, "ane_get_state")
		purego.RegisterLibFunc(&cSetState, lib, "ane_set_state")
		purego.RegisterLibFunc(&cImport, lib, "ane_import_tensor")
		purego.RegisterLibFunc(&cExport, lib, "ane_export_tensor")
		purego.RegisterLibFunc(&cTensorSize, lib, "ane_tensor_size")
		purego.RegisterLibFunc(&cDecode, lib, "ane_decode_sample")
		purego.RegisterLibFunc(&cReseed, lib, "ane_reseed")
	})
	return loadErr
}

func cString(p *byte) string {
	if p == nil {
		return ""
	}
	n := 0
	for *(*byte)(unsafe.Add(unsafe.Pointer(p), n)) != 0 {
		n++
	}
	return string(unsafe.Slice(p, n))
}

// Engine holds only the opaque handle and cached scalars; all state lives on the device.
type Engine struct {
	h      uintptr
	seq    int
	vocab  int
	seed   int64 // Options.Seed after defaults: LoadCheckpoint reseeds the sampler with seed + meta.Step
	layers int
	stock  bool // the reference's fixed model (stories.* sizes, reference architecture): checkpoints apply
}

func (e *Engine) err(op string, rc int32) error {
	return fmt.Errorf("storiesane %s: %s (status %d)", op, cString(cLastError(e.h)), rc)
}

// stockModel reports whether the options describe the model the stories package is compiled for
// (ane/stories/config.go:3-18) in the reference architecture: only then can its files be loaded.
func stockModel(o Options) bool {
	is := func(v, want int) bool { return v == 0 || v == want }
	return o.Arch == 0 && is(o.Dim, stories.Dim) && is(o.Hidden, stories.Hidden) && is(o.Layers, stories.NLayers) &&
		is(o.Heads, stories.Heads) && is(o.KVHeads, stories.Heads) && is(o.Vocab, stories.Vocab)
}

// Open mirrors ane.Open (ane/engine.go:184-355): ModelPath is required and is read as a llama2.c model
// file, else as a training checkpoint (weights and optimizer state), exactly like ane/engine.go:250-257.
func Open(opts Options) (*Engine, error) {
	if opts.ModelPath == "" && !opts.NoModel {
		return nil, fmt.Errorf("storiesane open: model path is empty") // ane/engine.go:185-187
	}
	if opts.ModelPath != "" && !stockModel(opts) {
		return nil, fmt.Errorf("storiesane open: model files describe the %d-dim reference model; use NoModel and ImportTensor for other shapes", stories.Dim)
	}
	if err := load(); err != nil {
		return nil, err
	}
	seq := opts.Seq
	if seq <= 0 {
		seq = 256
	}
	if len(opts.Tokens) > 0 && len(opts.Tokens) < seq+1 {
		return nil, fmt.Errorf("storiesane open: not enough tokens for seq=%d", seq)
	}
	co := cOptions{
		dim: int32(opts.Dim), hidden: int32(opts.Hidden), nLayers: int32(opts.Layers), nHeads: int32(opts.Heads),
		nKVHeads: int32(opts.KVHeads), vocab: int32(opts.Vocab), seq: int32(opts.Seq), batch: int32(opts.Batch),
		arch: int32(opts.Arch), accumSteps: int32(opts.AccumSteps), lr: opts.LR, seed: opts.Seed,
		beta1: opts.AdamBeta1, beta2: opts.AdamBeta2, eps: opts.AdamEps, weightDecay: opts.WeightDecay,
		gradClip: opts.GradClip, lossSc: opts.LossScale, embedLRMult: opts.EmbedLRMult,
		scalarLRMult: opts.ScalarLRMult, lambdaLRMult: opts.LambdaLRMult, lambdaBeta1: opts.LambdaBeta1,
		lambdaBeta2: opts.LambdaBeta2, device: int32(opts.Device), rank: int32(opts.Rank),
		worldSize: int32(opts.WorldSize),
	}
	co.structSize = uint32(unsafe.Sizeof(co))
	if !opts.ExactGradients {
		co.quirks = 1
	}
	if opts.FP32 {
		co.computeDtype = 1
	}
	var tokPtr *uint16
	if len(opts.Tokens) > 0 {
		tokPtr = unsafe.SliceData(opts.Tokens)
	}
	var dpPtr *byte
	if len(opts.DPID) == 128 {
		dpPtr = unsafe.SliceData(opts.DPID)
	}
	var h uintptr
	rc := cOpen(&co, tokPtr, uint64(len(opts.Tokens)), dpPtr, &h)
	runtime.KeepAlive(opts.Tokens)
	runtime.KeepAlive(opts.DPID)
	if rc != 0 {
		return nil, fmt.Errorf("storiesane open: %s (status %d)", cString(cLastError(0)), rc)
	}
	vocab := opts.Vocab
	if vocab <= 0 {
		vocab = stories.Vocab
	}
	layers := opts.Layers
	if layers <= 0 {
		layers = stories.NLayers
	}
	seed := opts.Seed
	if seed == 0 {
		seed = 42 // ane/engine.go:200-202
	}
	e := &Engine{h: h, seq: seq, vocab: vocab, seed: seed, layers: layers, stock: stockModel(opts)}
	if opts.ModelPath != "" {
		// ane/engine.go:248-257: pretrained file first, checkpoint second; the first error is the one reported
		mw := stories.NewModelWeights(stories.Vocab)
		var opt *stories.OptimState
		if len(opts.Tokens) > 0 {
			opt = stories.NewOptimState(stories.Vocab)
		}
		loaded, _, err := stories.LoadPretrained(opts.ModelPath)
		if err != nil {
			if _, ckptErr := stories.LoadCheckpoint(opts.ModelPath, mw, opt); ckptErr != nil {
				e.Close()
				return nil, fmt.Errorf("storiesane open: load model: %w", err)
			}
		} else {
			*mw = *loaded
			opt = nil // a model file carries no optimizer state: the device moments stay zero
		}
		if err := e.pushModel(mw, opt); err != nil {
			e.Close()
			return nil, err
		}
	}
	return e, nil
}

// Close mirrors (*Engine).Close (ane/engine.go:567).
func (e *Engine) Close() {
	if e == nil || e.h == 0 {
		return
	}
	cClose(e.h)
	e.h = 0
}

// Prepare is a no-op: nothing is compiled at run time (ane/runtime.go:10).
func (e *Engine) Prepare() {}

// SetGradTaskConcurrency is accepted for source compatibility (ane/common.go:17).
func SetGradTaskConcurrency(int) {}

// Step mirrors (*Engine).Step (ane/engine.go:381).
func (e *Engine) Step() (StepResult, error) {
	if e == nil || e.h == 0 {
		return StepResult{}, fmt.Errorf("storiesane step: engine is closed")
	}
	var r cStepResult
	r.structSize = uint32(unsafe.Sizeof(r))
	if rc := cStep(e.h, &r); rc != 0 {
		return StepResult{}, e.err("step", rc)
	}
	return StepResult{
		Loss:            r.loss,
		StepDuration:    time.Duration(r.stepNS),
		ANEEvalDuration: time.Duration(r.deviceEvalNS),
		CPUWorkDuration: time.Duration(r.cpuWorkNS),
		AdamDuration:    time.Duration(r.adamNS),
	}, nil
}

// EvalLogits mirrors (*Engine).EvalLogits (ane/engine.go:449): len(tokens) must equal seq; the
// result is a fresh slice of vocab*seq floats in [v*seq+t] order.
func (e *Engine) EvalLogits(tokens []uint16) ([]float32, error) {
	if e == nil || e.h == 0 {
		return nil, fmt.Errorf("storiesane eval logits: engine is closed")
	}
	if len(tokens) != e.seq {
		return nil, fmt.Errorf("storiesane eval logits: token len=%d want=%d", len(tokens), e.seq)
	}
	out := make([]float32, e.vocab*e.seq)
	rc := cEvalLogits(e.h, unsafe.SliceData(tokens), 1, unsafe.SliceData(out), uint64(len(out)), 0)
	runtime.KeepAlive(tokens)
	if rc != 0 {
		return nil, e.err("eval logits", rc)
	}
	return out, nil
}

// EvalLogitsInto is EvalLogits into a caller-owned slice of vocab*seq values (not in the reference: its
// EvalLogits returns a fresh slice, ane/engine.go:449-462).  Into a slice from HostAlloc the logits come straight
// from the device (1.39 against 1.67 ms per 32000 x 256 window measured through the Python twin of this call).
func (e *Engine) EvalLogitsInto(tokens []uint16, dst []float32) error {
	if e == nil || e.h == 0 {
		return fmt.Errorf("storiesane eval logits: engine is closed")
	}
	if len(tokens) != e.seq {
		return fmt.Errorf("storiesane eval logits: token len=%d want=%d", len(tokens), e.seq)
	}
	if len(dst) < e.vocab*e.seq {
		return fmt.Errorf("storiesane eval logits: dst len=%d want=%d", len(dst), e.vocab*e.seq)
	}
	rc := cEvalLogits(e.h, unsafe.SliceData(tokens), 1, unsafe.SliceData(dst), uint64(len(dst)), 0)
	runtime.KeepAlive(tokens)
	runtime.KeepAlive(dst)
	if rc != 0 {
		return e.err("eval logits", rc)
	}
	return nil
}

// HostAlloc returns n float32 of page-locked host memory outside the Go heap and the function that releases it.
func HostAlloc(n int) ([]float32, func(), error) {
	if err := load(); err != nil {
		return nil, nil, err
	}
	p := cHostMalloc(uint64(n) * 4)
	if p == nil {
		return nil, nil, fmt.Errorf("storiesane host alloc: %d bytes of page-locked memory not available", n*4)
	}
	return unsafe.Slice((*float32)(p), n), func() { cHostFree(p) }, nil
}

// EvalLoss is additive: the summed next-token negative log-likelihood of one window and the
// number of scored positions, computed on the device.
func (e *Engine) EvalLoss(tokens []uint16) (float64, int, error) {
	if e == nil || e.h == 0 {
		return 0, 0, fmt.Errorf("storiesane eval loss: engine is closed")
	}
	if len(tokens) != e.seq {
		return 0, 0, fmt.Errorf("storiesane eval loss: token len=%d want=%d", len(tokens), e.seq)
	}
	var sum float64
	var n uint64
	rc := cEvalLoss(e.h, unsafe.SliceData(tokens), 1, &sum, &n)
	runtime.KeepAlive(tokens)
	if rc != 0 {
		return 0, 0, e.err("eval loss", rc)
	}
	return sum, int(n), nil
}

// Generate is additive: KV-cached generation for nSeq prompts of equal length laid out back to back.
// temperature <= 1e-6 is the reference's argmax (ane/train_full.go:344-354); otherwise its
// sampleFromLogits (ane/train_full.go:318-342) with rng.Float64() drawn here, one draw per token in
// step-major order, so a caller that seeds rng like the reference reproduces its choices.
func (e *Engine) Generate(rng *rand.Rand, prompts []uint16, nSeq, nNew int, temperature float32) ([]uint16, error) {
	if e == nil || e.h == 0 {
		return nil, fmt.Errorf("storiesane decode: engine is closed")
	}
	if nSeq <= 0 || nNew <= 0 || len(prompts) == 0 || len(prompts)%nSeq != 0 {
		return nil, fmt.Errorf("storiesane decode: prompts len=%d not a multiple of nSeq=%d", len(prompts), nSeq)
	}
	var draws []float64
	if temperature > 1e-6 {
		if rng == nil {
			return nil, fmt.Errorf("storiesane decode: sampling needs a rand source")
		}
		draws = make([]float64, nSeq*nNew)
		for i := range draws {
			draws[i] = rng.Float64()
		}
	}
	out := make([]uint16, nSeq*nNew)
	rc := cDecode(e.h, unsafe.SliceData(prompts), uint32(nSeq), uint32(len(prompts)/nSeq), uint32(nNew), temperature,
		unsafe.SliceData(draws), unsafe.SliceData(out))
	runtime.KeepAlive(prompts)
	runtime.KeepAlive(draws)
	if rc != 0 {
		return nil, e.err("decode", rc)
	}
	return out, nil
}

// Flush mirrors (*Engine).Flush (ane/engine.go:484).
func (e *Engine) Flush() (time.Duration, error) {
	if e == nil || e.h == 0 {
		return 0, fmt.Errorf("storiesane flush: engine is closed")
	}
	var ms float64
	if rc := cFlush(e.h, &ms); rc != 0 {
		return 0, e.err("flush", rc)
	}
	return time.Duration(ms * float64(time.Millisecond)), nil
}

// LR mirrors (*Engine).LR (ane/engine.go:358).
func (e *Engine) LR() float32 {
	if e == nil || e.h == 0 {
		return 0
	}
	return cGetLR(e.h)
}

// SetLR mirrors (*Engine).SetLR (ane/engine.go:366).
func (e *Engine) SetLR(lr float32) error {
	if e == nil || e.h == 0 {
		return fmt.Errorf("storiesane set lr: engine is closed")
	}
	if lr <= 0 {
		return fmt.Errorf("storiesane set lr: lr must be > 0")
	}
	if rc := cSetLR(e.h, lr); rc != 0 {
		return e.err("set lr", rc)
	}
	return nil
}

// State mirrors (*Engine).State (ane/engine.go:498).
func (e *Engine) State() State {
	if e == nil || e.h == 0 {
		return State{}
	}
	var s cState
	s.structSize = uint32(unsafe.Sizeof(s))
	if cGetState(e.h, &s) != 0 {
		return State{}
	}
	return State{TokenPos: s.tokenPos, LastLoss: s.lastLoss, CumTrainMS: s.cumTrainMS, CumWallMS: s.cumWallMS,
		CumSteps: s.cumSteps, CumBatches: s.cumBatches, AdamT: s.adamT, PendingSteps: s.pendingSteps}
}

// LoadState mirrors (*Engine).LoadState (ane/engine.go:506).
func (e *Engine) LoadState(st State) error {
	if e == nil || e.h == 0 {
		return fmt.Errorf("storiesane load state: engine is closed")
	}
	s := cState{tokenPos: st.TokenPos, lastLoss: st.LastLoss, cumTrainMS: st.CumTrainMS, cumWallMS: st.CumWallMS,
		cumSteps: st.CumSteps, cumBatches: st.CumBatches, adamT: st.AdamT, pendingSteps: st.PendingSteps}
	s.structSize = uint32(unsafe.Sizeof(s))
	if rc := cSetState(e.h, &s); rc != 0 {
		return e.err("load state", rc)
	}
	return nil
}

// ImportTensor / ExportTensor move one tensor (reference shapes, ane/stories/weights.go:13-42)
// between Go slices and the device; which: 0 weight, 1 gradient, 2 Adam m, 3 Adam v.
func (e *Engine) ImportTensor(id, layer, which uint32, data []float32) error {
	if e == nil || e.h == 0 {
		return fmt.Errorf("storiesane import: engine is closed")
	}
	rc := cImport(e.h, id, layer, which, unsafe.SliceData(data), uint64(len(data)))
	runtime.KeepAlive(data)
	if rc != 0 {
		return e.err("import", rc)
	}
	return nil
}

func (e *Engine) ExportTensor(id, layer, which uint32) ([]float32, error) {
	if e == nil || e.h == 0 {
		return nil, fmt.Errorf("storiesane export: engine is closed")
	}
	n := cTensorSize(e.h, id, layer)
	if n <= 0 {
		return nil, nil
	}
	out := make([]float32, n)
	if rc := cExport(e.h, id, layer, which, unsafe.SliceData(out), uint64(n)); rc != 0 {
		return nil, e.err("export", rc)
	}
	return out, nil
}
