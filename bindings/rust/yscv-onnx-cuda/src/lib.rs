//! The `yscv-onnx` side of the boundary: what `crates/yscv-onnx/src/runner/cuda.rs` would hold
//! behind a `cuda` feature, following the pattern of the existing `#[cfg(feature = "gpu")]`
//! runner (runner/gpu/mod.rs:1379-1441): a load-time hook that uploads weights once, and the
//! three handlers `exec_matmul` (int4 branch), `exec_qlinear_matmul`, `exec_matmul_integer`
//! (runner/linear.rs:223-278, 438-537, 648-737) calling the library instead of the CPU kernels.
//!
//! The reference's tensors are f32 even for integer data (loader/convert.rs:14-48); the
//! handlers convert to bytes per call exactly where the reference does (linear.rs:462, 674).
//! Written against a minimal view of the runner's types so that it compiles on its own:
//! `TensorView` stands for `yscv_tensor::Tensor`, `OnnxError` for `crate::error::OnnxError`.
use yscv_kernels_cuda::{self as cuda, Context, CudaError, Rounding, WeightLayout, WeightRegistry};

/// What the handlers need of `yscv_tensor::Tensor`.
pub struct TensorView<'a> {
    pub shape: &'a [usize],
    pub data: &'a [f32],
}

#[derive(Debug)]
pub enum OnnxError {
    /// `OnnxError::DecodeFailed { message }` (shape mismatches, runner/linear.rs:470-475)
    DecodeFailed { message: String },
    /// `OnnxError::MissingInput` (runner/dispatch.rs:12-15)
    MissingInput { name: String },
    /// `KernelError::Gpu { message }` -> `OnnxError::GpuKernel` (crates/yscv-onnx/src/error.rs:35-41)
    GpuKernel { message: String },
}

impl From<CudaError> for OnnxError {
    fn from(e: CudaError) -> Self {
        OnnxError::GpuKernel { message: e.to_string() }
    }
}

/// A weight initializer as `build_runtime_index` sees it (plan/build.rs:1417-1454).
pub enum Initializer<'a> {
    /// MatMul / Gemm fp32 weight to be packed to int4 (`quantize_matmul_weights_int4_packed`)
    MatMulF32 { data: &'a [f32], dims: [usize; 2], layout: WeightLayout },
    /// QLinearMatMul input 3 / MatMulInteger input 1, rank 2, f32-encoded integers
    Int8 { data: &'a [f32], k: usize, n: usize },
}

/// Load-time hook: uploads every eligible weight once and records it under its initializer
/// name. Returns (int4 weights packed, int8 weights prepacked), the counts
/// `quantize_matmul_weights_int4_packed` and the prepack loop report.
pub fn upload_weights<'a>(ctx: &mut Context, reg: &WeightRegistry, group_size: usize,
                          weights: impl IntoIterator<Item = (&'a str, Initializer<'a>)>)
                          -> Result<(usize, usize), OnnxError> {
    let (mut packed, mut prepacked) = (0, 0);
    for (name, init) in weights {
        match init {
            Initializer::MatMulF32 { data, dims, layout } => {
                if reg.register_matmul_weight(ctx, name, data, dims, layout, group_size)? {
                    packed += 1; // the fp32 initializer can now be dropped (packed_int4.rs:120)
                }
            }
            Initializer::Int8 { data, k, n } => {
                // tensor_data_as_i8 (plan/build.rs:1367-1369): round, then the saturating cast
                let bytes: Vec<i8> = data.iter().map(|v| v.round() as i8).collect();
                if reg.register_i8_weight(ctx, name, &bytes, k, n)? {
                    prepacked += 1;
                }
            }
        }
    }
    Ok((packed, prepacked))
}

/// `exec_matmul`, int4 branch (runner/linear.rs:223-278): the weight is looked up by the name
/// of input 1; leading dimensions of the activation flatten into M; one library call replaces
/// the `GEMM_THRESHOLD` split (the library reads the weights once for any M).
/// Returns `Ok(None)` when the name is not in the table: the caller takes its fp32 path.
pub fn exec_matmul_int4(ctx: &mut Context, reg: &WeightRegistry, weight_name: &str, a: &TensorView<'_>)
                        -> Result<Option<(Vec<usize>, Vec<f32>)>, OnnxError> {
    let Some(w) = reg.int4(weight_name) else { return Ok(None) };
    let rank = a.shape.len();
    if rank < 2 || a.shape[rank - 1] != w.k() {
        return Err(OnnxError::DecodeFailed {
            message: format!("MatMul int4: activation shape {:?} does not end in k = {}", a.shape, w.k()),
        });
    }
    let m: usize = a.shape[..rank - 1].iter().product();
    let mut out = vec![0f32; m * w.rows()];
    w.matmul(ctx, a.data, &mut out, m)?;
    let mut shape = a.shape[..rank - 1].to_vec();
    shape.push(w.rows());
    Ok(Some((shape, out)))
}

fn scalar(t: &TensorView<'_>) -> f32 {
    t.data[0] // only `.data()[0]` is read: per-tensor semantics (runner/linear.rs:440-446)
}

/// f32-encoded integers -> bytes; `unsigned` selects the uint8 or the int8 reading.
fn to_bytes(t: &TensorView<'_>, unsigned: bool) -> Vec<u8> {
    if unsigned {
        t.data.iter().map(|&v| v as u8).collect()
    } else {
        t.data.iter().map(|&v| (v as i8) as u8).collect()
    }
}

/// `exec_qlinear_matmul` (runner/linear.rs:438-537). The reference takes its integer kernel only
/// when both zero points are 0 and falls back to an fp32 GEMM otherwise; here any zero point is
/// exact in integers. `uint8_io` selects the ONNX uint8 contract (round half to even, [0, 255])
/// instead of the runner's int8 one (`f32::round`, [-128, 127], linear.rs:481-485).
#[allow(clippy::too_many_arguments)]
pub fn exec_qlinear_matmul(ctx: &mut Context, reg: &WeightRegistry, weight_name: &str, a: &TensorView<'_>,
                           a_scale: &TensorView<'_>, a_zp: &TensorView<'_>, b_scale: &TensorView<'_>,
                           y_scale: &TensorView<'_>, y_zp: &TensorView<'_>, uint8_io: bool)
                           -> Result<(Vec<usize>, Vec<f32>), OnnxError> {
    // (a view: the table keeps the handle)
    let view = reg.i8b(weight_name).ok_or_else(|| OnnxError::MissingInput { name: weight_name.to_string() })?;
    if a.shape.len() != 2 {
        return Err(OnnxError::DecodeFailed { message: format!("QLinearMatMul needs rank 2, got {:?}", a.shape) });
    }
    let (m, k) = (a.shape[0], a.shape[1]);
    if k != view.k() {
        return Err(OnnxError::DecodeFailed { message: format!("QLinearMatMul: k = {k}, weight has {}", view.k()) });
    }
    let composite = (scalar(a_scale) * scalar(b_scale)) / scalar(y_scale); // f32, as linear.rs:481
    let bytes = to_bytes(a, uint8_io);
    let mut out = vec![0u8; m * view.n()];
    let (qmin, qmax, rounding) = if uint8_io { (0, 255, Rounding::TiesToEven) } else { (-128, 127, Rounding::HalfAwayFromZero) };
    cuda::qlinear_matmul(ctx, &bytes, uint8_io, scalar(a_zp) as i32, &view, m, composite, scalar(y_zp), qmin, qmax,
                         rounding, &mut out)?;
    let as_f32 = if uint8_io { out.iter().map(|&q| q as f32).collect() } else { out.iter().map(|&q| (q as i8) as f32).collect() };
    Ok((vec![m, view.n()], as_f32))
}

/// `exec_matmul_integer` (runner/linear.rs:648-737): exact for any zero points (the reference
/// leaves its integer path when either is non-zero, linear.rs:701-735). The zero point of B is a
/// property of the prepacked handle, set once at load time.
pub fn exec_matmul_integer(ctx: &mut Context, reg: &WeightRegistry, weight_name: &str, a: &TensorView<'_>,
                           a_zp: Option<&TensorView<'_>>, a_is_uint8: bool)
                           -> Result<(Vec<usize>, Vec<f32>), OnnxError> {
    let view = reg.i8b(weight_name).ok_or_else(|| OnnxError::MissingInput { name: weight_name.to_string() })?;
    if a.shape.len() != 2 {
        return Err(OnnxError::DecodeFailed { message: format!("MatMulInteger needs rank 2, got {:?}", a.shape) });
    }
    let m = a.shape[0];
    let bytes = to_bytes(a, a_is_uint8);
    let mut acc = vec![0i32; m * view.n()];
    cuda::matmul_integer(ctx, &bytes, a_is_uint8, a_zp.map_or(0, |t| scalar(t) as i32), &view, m, &mut acc)?;
    Ok((vec![m, view.n()], acc.iter().map(|&v| v as f32).collect())) // i32 carried as f32 (linear.rs:693)
}
