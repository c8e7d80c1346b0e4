// Checkpoints of the Go engine: (*Engine).SaveCheckpoint / LoadCheckpoint of the reference
// (ane/engine.go:515-565) over device-resident state.  The file body is written and read by the untouched
// stories package (stories.SaveCheckpoint / stories.LoadCheckpoint, ane/stories/ckpt.go:77-405); tensors
// cross to the device with ExportTensor / ImportTensor; the "SANE" trailer (ane/engine.go:684-765: token
// position, pending micro-steps, accumulated gradients) is written and read here in the reference's layout.
//
// Like engine.go this file cannot be compiled in the build container (no Go toolchain).
package ane

import (
	"encoding/binary"
	"fmt"
	"io"
	"os"

	"github.com/tmc/autoresearch-go-ane/ane/stories"
)

// Tensor ids of include/ane_b200.h.
const (
	tEmbed = iota
	tWQ
	tWK
	tWV
	tWO
	tW1
	tW2
	tW3
	tRMSAtt
	tRMSFFN
	tRMSFinal
	tVEEmbed
	tVEGate
	tResidLambdas
	tX0Lambdas
	tSmearGate
	tSmearLambda
	tBackoutLambda
)

// which-codes of ane_import_tensor / ane_export_tensor.
const (
	kWeight = iota
	kGrad
	kAdamM
	kAdamV
)

const (
	trailerMagic     = "SANE" // ane/engine.go:685
	trailerVersionV1 = uint32(1)
	trailerVersionV2 = uint32(2)
)

// layerSlices lists one layer's tensors in checkpoint order (ane/stories/ckpt.go:162-199,
// ane/engine.go:811-823) with their tensor ids.
func layerSlices(l *stories.LayerWeights) ([]uint32, [][]float32) {
	return []uint32{tWQ, tWK, tWV, tWO, tW1, tW2, tVEEmbed, tVEGate},
		[][]float32{l.Wq, l.Wk, l.Wv, l.Wo, l.W1, l.W2, l.VEEmbed, l.VEGate}
}

func layerAdam(l *stories.LayerOptimState) []*stories.AdamState {
	return []*stories.AdamState{&l.Wq, &l.Wk, &l.Wv, &l.Wo, &l.W1, &l.W2, &l.VEEmbed, &l.VEGate}
}

func modelSlices(mw *stories.ModelWeights) ([]uint32, [][]float32) {
	return []uint32{tEmbed, tResidLambdas, tX0Lambdas, tSmearGate, tSmearLambda, tBackoutLambda},
		[][]float32{mw.Embed, mw.ResidLambdas, mw.X0Lambdas, mw.SmearGate, mw.SmearLambda, mw.BackoutLambda}
}

func modelAdam(opt *stories.OptimState) []*stories.AdamState {
	return []*stories.AdamState{&opt.Embed, &opt.ResidLambdas, &opt.X0Lambdas, &opt.SmearGate, &opt.SmearLambda, &opt.BackoutLambda}
}

// pushModel sends weights (and, when opt is given, Adam moments) to the device.
func (e *Engine) pushModel(mw *stories.ModelWeights, opt *stories.OptimState) error {
	put := func(id uint32, layer int, which uint32, v []float32) error {
		if len(v) == 0 {
			return nil // value-embedding tensors of layers that have none
		}
		return e.ImportTensor(id, uint32(layer), which, v)
	}
	for i := range mw.Layers {
		ids, ws := layerSlices(&mw.Layers[i])
		for k := range ids {
			if err := put(ids[k], i, kWeight, ws[k]); err != nil {
				return err
			}
		}
		if opt != nil {
			for k, st := range layerAdam(&opt.Layers[i]) {
				if err := put(ids[k], i, kAdamM, st.M); err != nil {
					return err
				}
				if err := put(ids[k], i, kAdamV, st.V); err != nil {
					return err
				}
			}
		}
	}
	ids, ws := modelSlices(mw)
	for k := range ids {
		if err := put(ids[k], 0, kWeight, ws[k]); err != nil {
			return err
		}
	}
	if opt != nil {
		for k, st := range modelAdam(opt) {
			if err := put(ids[k], 0, kAdamM, st.M); err != nil {
				return err
			}
			if err := put(ids[k], 0, kAdamV, st.V); err != nil {
				return err
			}
		}
	}
	return nil
}

// pullInto fills dst (already sized by the stories constructors) from the device.
func (e *Engine) pullInto(id uint32, layer int, which uint32, dst []float32) error {
	if len(dst) == 0 {
		return nil
	}
	got, err := e.ExportTensor(id, uint32(layer), which)
	if err != nil {
		return err
	}
	if len(got) != len(dst) {
		return fmt.Errorf("storiesane export: tensor %d layer %d has %d elements, want %d", id, layer, len(got), len(dst))
	}
	copy(dst, got)
	return nil
}

func (e *Engine) pullModel(mw *stories.ModelWeights, opt *stories.OptimState) error {
	for i := range mw.Layers {
		ids, ws := layerSlices(&mw.Layers[i])
		adam := layerAdam(&opt.Layers[i])
		for k := range ids {
			if err := e.pullInto(ids[k], i, kWeight, ws[k]); err != nil {
				return err
			}
			if err := e.pullInto(ids[k], i, kAdamM, adam[k].M); err != nil {
				return err
			}
			if err := e.pullInto(ids[k], i, kAdamV, adam[k].V); err != nil {
				return err
			}
		}
	}
	ids, ws := modelSlices(mw)
	adam := modelAdam(opt)
	for k := range ids {
		if err := e.pullInto(ids[k], 0, kWeight, ws[k]); err != nil {
			return err
		}
		if err := e.pullInto(ids[k], 0, kAdamM, adam[k].M); err != nil {
			return err
		}
		if err := e.pullInto(ids[k], 0, kAdamV, adam[k].V); err != nil {
			return err
		}
	}
	return nil
}

// gradOrder visits the accumulated gradients in trailer order (writeModelGrad, ane/engine.go:811-840).
func (e *Engine) gradOrder(visit func(id uint32, layer int, n int) error) error {
	for i := 0; i < e.layers; i++ {
		for _, id := range []uint32{tWQ, tWK, tWV, tWO, tW1, tW2, tVEEmbed, tVEGate} { // sizes come from the device
			n := cTensorSize(e.h, id, uint32(i))
			if n > 0 {
				if err := visit(id, i, int(n)); err != nil {
					return err
				}
			}
		}
	}
	for _, id := range []uint32{tEmbed, tResidLambdas, tX0Lambdas, tSmearGate, tSmearLambda, tBackoutLambda} {
		n := cTensorSize(e.h, id, 0)
		if n > 0 {
			if err := visit(id, 0, int(n)); err != nil {
				return err
			}
		}
	}
	return nil
}

// SaveCheckpoint mirrors (*Engine).SaveCheckpoint (ane/engine.go:515-532).
func (e *Engine) SaveCheckpoint(path string, meta stories.TrainMeta) error {
	if e == nil || e.h == 0 {
		return fmt.Errorf("storiesane save checkpoint: engine is closed")
	}
	if !e.stock {
		return fmt.Errorf("storiesane save checkpoint: the V5 file describes the reference model only")
	}
	st := e.State()
	meta.LR = e.LR()
	meta.Loss = st.LastLoss
	meta.CumTrain = st.CumTrainMS
	meta.CumWall = st.CumWallMS
	meta.CumSteps = int(st.CumSteps)
	meta.CumBatches = int(st.CumBatches)
	meta.AdamT = int(st.AdamT)
	mw := stories.NewModelWeights(stories.Vocab)
	opt := stories.NewOptimState(stories.Vocab)
	if err := e.pullModel(mw, opt); err != nil {
		return err
	}
	if err := stories.SaveCheckpoint(path, meta, mw, opt); err != nil {
		return err
	}
	return e.appendTrailer(path, st)
}

// appendTrailer mirrors ane/engine.go:690-716; the device always holds accumulation buffers, so the
// trailer is version 2.
func (e *Engine) appendTrailer(path string, st State) error {
	f, err := os.OpenFile(path, os.O_WRONLY|os.O_APPEND, 0)
	if err != nil {
		return fmt.Errorf("storiesane append trailer: %w", err)
	}
	defer f.Close()
	if _, err := f.Write([]byte(trailerMagic)); err != nil {
		return fmt.Errorf("storiesane append trailer: write magic: %w", err)
	}
	for _, v := range []any{trailerVersionV2, st.TokenPos, st.PendingSteps} {
		if err := binary.Write(f, binary.LittleEndian, v); err != nil {
			return fmt.Errorf("storiesane append trailer: %w", err)
		}
	}
	return e.gradOrder(func(id uint32, layer int, n int) error {
		g, err := e.ExportTensor(id, uint32(layer), kGrad)
		if err != nil {
			return fmt.Errorf("storiesane append trailer: write accum grads: %w", err)
		}
		return binary.Write(f, binary.LittleEndian, g)
	})
}

// LoadCheckpoint mirrors (*Engine).LoadCheckpoint (ane/engine.go:534-565): weights, moments, learning
// rate and counters from the file, pending gradients cleared and then restored from the trailer, the
// sampler restarted at seed + meta.Step, the wall clock continued from meta.CumWall.
func (e *Engine) LoadCheckpoint(path string) (stories.TrainMeta, error) {
	if e == nil || e.h == 0 {
		return stories.TrainMeta{}, fmt.Errorf("storiesane load checkpoint: engine is closed")
	}
	if !e.stock {
		return stories.TrainMeta{}, fmt.Errorf("storiesane load checkpoint: the V5 file describes the reference model only")
	}
	mw := stories.NewModelWeights(stories.Vocab)
	opt := stories.NewOptimState(stories.Vocab)
	meta, err := stories.LoadCheckpoint(path, mw, opt)
	if err != nil {
		return stories.TrainMeta{}, err
	}
	if err := e.pushModel(mw, opt); err != nil {
		return stories.TrainMeta{}, err
	}
	if meta.LR > 0 {
		if err := e.SetLR(meta.LR); err != nil {
			return stories.TrainMeta{}, err
		}
	}
	st := State{LastLoss: meta.Loss, CumTrainMS: meta.CumTrain, CumWallMS: meta.CumWall,
		CumSteps: uint32(meta.CumSteps), CumBatches: uint32(meta.CumBatches), AdamT: uint32(meta.AdamT)}
	size, err := e.bodySize()
	if err != nil {
		return stories.TrainMeta{}, err
	}
	if err := e.loadTrailer(path, size, &st); err != nil {
		return stories.TrainMeta{}, err
	}
	if err := e.LoadState(st); err != nil { // also restarts the wall clock at now - CumWall
		return stories.TrainMeta{}, err
	}
	if rc := cReseed(e.h, e.seed+int64(meta.Step)); rc != 0 { // ane/engine.go:559
		return stories.TrainMeta{}, e.err("load checkpoint", rc)
	}
	return meta, nil
}

// bodySize is storiesCheckpointSize (ane/engine.go:767-791): header plus weights, moments and model-level
// tensors, i.e. the offset of the trailer.
func (e *Engine) bodySize() (int64, error) {
	total := int64(0)
	err := e.gradOrder(func(id uint32, layer int, n int) error {
		total += 3 * int64(n) // weight + m + v
		return nil
	})
	return 96 + 4*total, err
}

// loadTrailer mirrors ane/engine.go:718-765.  A missing trailer or a foreign magic is not an error;
// pending gradients are zero in that case.
func (e *Engine) loadTrailer(path string, offset int64, st *State) error {
	f, err := os.Open(path)
	if err != nil {
		return fmt.Errorf("storiesane load trailer: %w", err)
	}
	defer f.Close()
	if _, err := f.Seek(offset, io.SeekStart); err != nil {
		return fmt.Errorf("storiesane load trailer: seek: %w", err)
	}
	haveGrads := false
	var magic [4]byte
	if _, err := io.ReadFull(f, magic[:]); err == nil && string(magic[:]) == trailerMagic {
		var ver uint32
		if err := binary.Read(f, binary.LittleEndian, &ver); err != nil {
			return fmt.Errorf("storiesane load trailer: read version: %w", err)
		}
		if err := binary.Read(f, binary.LittleEndian, &st.TokenPos); err != nil {
			return fmt.Errorf("storiesane load trailer: read token pos: %w", err)
		}
		if err := binary.Read(f, binary.LittleEndian, &st.PendingSteps); err != nil {
			return fmt.Errorf("storiesane load trailer: read pending steps: %w", err)
		}
		switch ver {
		case trailerVersionV1: // carries two buffers that no longer exist; nothing to restore
		case trailerVersionV2:
			haveGrads = true
		default:
			return fmt.Errorf("storiesane load trailer: unsupported version %d", ver)
		}
	} else if err != nil && err != io.EOF && err != io.ErrUnexpectedEOF {
		return fmt.Errorf("storiesane load trailer: read magic: %w", err)
	}
	return e.gradOrder(func(id uint32, layer int, n int) error {
		g := make([]float32, n) // zeros clear the device accumulator (ane/engine.go:550-555)
		if haveGrads {
			if err := binary.Read(f, binary.LittleEndian, g); err != nil {
				return fmt.Errorf("storiesane load trailer: read accum grads: %w", err)
			}
		}
		return e.ImportTensor(id, uint32(layer), kGrad, g)
	})
}
