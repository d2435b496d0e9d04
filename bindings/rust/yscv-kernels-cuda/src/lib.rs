//! Safe wrappers with the signatures of the `yscv_kernels` free functions they replace
//! (crates/yscv-kernels/src/core.rs:173-186, 230-235). Meant to live in yscv-kernels as
//! `src/cuda.rs` behind a `cuda` cargo feature, next to the existing `gpu` feature.
//!
//! The reference's kernels are infallible: shape errors are `debug_assert!`
//! (int4_matmul.rs:53-59, int8_matmul.rs:2408-2410). The wrappers keep that contract:
//! they validate what the reference asserts, call the library, and panic with the library's
//! message on a non-zero status. Callers that want a `Result` use the `try_` forms, whose
//! error maps onto `KernelError::Gpu { message }` (crates/yscv-kernels/src/error.rs:213-214).
use std::ffi::{CStr, CString};
use std::os::raw::c_int;
use std::ptr;
use std::sync::OnceLock;

use yscv_cuda_sys as sys;

/// A failed library call: the status code and the library's thread-local message.
#[derive(Debug, Clone)]
pub struct CudaError {
    pub status: i32,
    pub message: String,
}

impl std::fmt::Display for CudaError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "yscv_cuda status {}: {}", self.status, self.message)
    }
}
impl std::error::Error for CudaError {}

fn check(status: c_int) -> Result<(), CudaError> {
    if status == sys::YSCV_CUDA_OK {
        return Ok(());
    }
    // SAFETY: yscv_cuda_last_error returns a NUL-terminated string owned by the library,
    // valid until the calling thread's next failing call.
    let message = unsafe { CStr::from_ptr(sys::yscv_cuda_last_error()) }.to_string_lossy().into_owned();
    Err(CudaError { status, message })
}

/// One CUDA stream on one sm_100 device. Calls on one context are serialised by the caller
/// (`&mut self` on everything that enqueues work); contexts may live on different threads.
pub struct Context(*mut sys::yscv_cuda_ctx);

// SAFETY: the library keeps no thread affinity in a context; exclusive access is enforced by
// `&mut self`.
unsafe impl Send for Context {}

impl Context {
    pub fn new(device: i32) -> Result<Self, CudaError> {
        let mut raw = ptr::null_mut();
        // SAFETY: `raw` is a valid out-pointer.
        check(unsafe { sys::yscv_cuda_ctx_create(device, &mut raw) })?;
        Ok(Self(raw))
    }

    /// The device named by `YSCV_CUDA_DEVICE` (default 0), the counterpart of the reference's
    /// env-driven configuration (docs/env-vars.md).
    pub fn from_env() -> Result<Self, CudaError> {
        let device = std::env::var("YSCV_CUDA_DEVICE").ok().and_then(|v| v.parse().ok()).unwrap_or(0);
        Self::new(device)
    }

    pub fn raw(&mut self) -> *mut sys::yscv_cuda_ctx {
        self.0
    }

    /// Reads and clears the device status word (0 = no bounded wait gave up).
    pub fn device_status(&mut self) -> Result<i32, CudaError> {
        let mut s: c_int = 0;
        // SAFETY: valid context and out-pointer.
        check(unsafe { sys::yscv_cuda_ctx_device_status(self.0, &mut s) })?;
        Ok(s)
    }

    /// `runtime_dispatch_report()` for this context.
    pub fn dispatch_report(&self) -> String {
        // SAFETY: the returned string belongs to the calling thread until its next call.
        unsafe { CStr::from_ptr(sys::yscv_cuda_dispatch_report(self.0)) }.to_string_lossy().into_owned()
    }
}

impl Drop for Context {
    fn drop(&mut self) {
        // SAFETY: created by yscv_cuda_ctx_create, destroyed once.
        unsafe { sys::yscv_cuda_ctx_destroy(self.0) }
    }
}

thread_local! {
    // the reference's kernels are free functions: the drop-in forms below use one context per
    // calling thread (rayon workers, tower-parallel branches), created on first use
    static THREAD_CTX: std::cell::RefCell<Option<Context>> = const { std::cell::RefCell::new(None) };
}

fn with_ctx<R>(f: impl FnOnce(&mut Context) -> R) -> R {
    THREAD_CTX.with(|slot| {
        let mut slot = slot.borrow_mut();
        let ctx = slot.get_or_insert_with(|| Context::from_env().expect("no sm_100 device for yscv-cuda"));
        f(ctx)
    })
}

// ---- int4: drop-ins for int4_matmul.rs ------------------------------------------------------

/// `packed_int4_gemv_dispatch` (int4_matmul.rs:310-377).
pub fn packed_int4_gemv_dispatch(weight_packed: &[u8], scales: &[f32], activation: &[f32], output: &mut [f32],
                                 m_w: usize, k: usize, group_size: usize) {
    debug_assert_eq!(weight_packed.len(), m_w * k / 2);
    debug_assert_eq!(scales.len(), m_w * (k / group_size));
    debug_assert_eq!(activation.len(), k);
    debug_assert_eq!(output.len(), m_w);
    with_ctx(|ctx| {
        // SAFETY: slice lengths were checked against the shapes above.
        check(unsafe {
            sys::yscv_cuda_packed_int4_gemv(ctx.raw(), weight_packed.as_ptr(), scales.as_ptr(), activation.as_ptr(),
                                            output.as_mut_ptr(), m_w, k, group_size)
        })
        .expect("packed_int4_gemv")
    })
}

/// `packed_int4_gemm_dispatch` (int4_matmul.rs:548-605).
#[allow(clippy::too_many_arguments)]
pub fn packed_int4_gemm_dispatch(weight_packed: &[u8], scales: &[f32], activation: &[f32], output: &mut [f32],
                                 m: usize, n: usize, k: usize, group_size: usize) {
    debug_assert_eq!(weight_packed.len(), n * k / 2);
    debug_assert_eq!(activation.len(), m * k);
    debug_assert_eq!(output.len(), m * n);
    with_ctx(|ctx| {
        // SAFETY: as above.
        check(unsafe {
            sys::yscv_cuda_packed_int4_gemm(ctx.raw(), weight_packed.as_ptr(), scales.as_ptr(), activation.as_ptr(),
                                            output.as_mut_ptr(), m, n, k, group_size)
        })
        .expect("packed_int4_gemm")
    })
}

/// `pack_int4_symmetric_per_group` (int4_matmul.rs:611-646): bit-identical bytes and scales.
pub fn pack_int4_symmetric_per_group(weights: &[f32], m_w: usize, k: usize, group_size: usize) -> (Vec<u8>, Vec<f32>) {
    debug_assert_eq!(weights.len(), m_w * k);
    let mut packed = vec![0u8; m_w * k / 2];
    let mut scales = vec![0f32; m_w * (k / group_size)];
    with_ctx(|ctx| {
        // SAFETY: output vectors sized as the header asks.
        check(unsafe {
            sys::yscv_cuda_pack_int4_symmetric_per_group(ctx.raw(), weights.as_ptr(), m_w, k, group_size,
                                                         packed.as_mut_ptr(), scales.as_mut_ptr())
        })
        .expect("pack_int4")
    });
    (packed, scales)
}

/// `PackedInt4Weight` (crates/yscv-onnx/src/quantize/packed_int4.rs:28-39) resident in HBM.
pub struct ResidentInt4Weight {
    raw: *mut sys::yscv_cuda_int4_weight,
    owned: bool,
}
// SAFETY: handles are immutable after creation and may be shared between contexts.
unsafe impl Send for ResidentInt4Weight {}
unsafe impl Sync for ResidentInt4Weight {}

impl ResidentInt4Weight {
    pub fn upload(ctx: &mut Context, packed: &[u8], scales: &[f32], m_w: usize, k: usize, group_size: usize)
                  -> Result<Self, CudaError> {
        let mut raw = ptr::null_mut();
        // SAFETY: slices outlive the (synchronous) upload.
        check(unsafe {
            sys::yscv_cuda_int4_weight_upload(ctx.raw(), packed.as_ptr(), scales.as_ptr(), m_w, k, group_size, &mut raw)
        })?;
        Ok(Self { raw, owned: true })
    }
    pub fn rows(&self) -> usize { unsafe { sys::yscv_cuda_int4_weight_rows(self.raw) } }
    pub fn k(&self) -> usize { unsafe { sys::yscv_cuda_int4_weight_k(self.raw) } }
    pub fn group_size(&self) -> usize { unsafe { sys::yscv_cuda_int4_weight_group_size(self.raw) } }

    /// The int4 branch of `exec_matmul` (runner/linear.rs:223-278): activation [m, k] in host
    /// memory -> output [m, n]; one pass over the weights for any m.
    pub fn matmul(&self, ctx: &mut Context, activation: &[f32], output: &mut [f32], m: usize) -> Result<(), CudaError> {
        debug_assert_eq!(activation.len(), m * self.k());
        debug_assert_eq!(output.len(), m * self.rows());
        // SAFETY: lengths checked above.
        check(unsafe { sys::yscv_cuda_int4_matmul(ctx.raw(), self.raw, activation.as_ptr(), output.as_mut_ptr(), m) })
    }
}

impl Drop for ResidentInt4Weight {
    fn drop(&mut self) {
        if self.owned {
            // SAFETY: created by the library, freed once.
            unsafe { sys::yscv_cuda_int4_weight_free(self.raw) }
        }
    }
}

// ---- int8: drop-ins for int8_matmul.rs -------------------------------------------------------

/// `int8_matmul_dispatch` (int8_matmul.rs:2407-2413).
pub fn int8_matmul_dispatch(a: &[i8], b: &[i8], m: usize, k: usize, n: usize, out: &mut [i32]) {
    debug_assert_eq!(a.len(), m * k);
    debug_assert_eq!(b.len(), k * n);
    debug_assert_eq!(out.len(), m * n);
    with_ctx(|ctx| {
        // SAFETY: lengths checked above.
        check(unsafe { sys::yscv_cuda_int8_matmul(ctx.raw(), a.as_ptr(), b.as_ptr(), m, k, n, out.as_mut_ptr()) })
            .expect("int8_matmul")
    })
}

/// `PackedI8B` (int8_matmul.rs:128-160): the same accessors, the bytes live in HBM.
pub struct PackedI8B {
    raw: *mut sys::yscv_cuda_i8b,
    owned: bool, // false: a view of a handle the registry owns
}
// SAFETY: immutable after creation (the zero point is set before the handle is shared).
unsafe impl Send for PackedI8B {}
unsafe impl Sync for PackedI8B {}

impl PackedI8B {
    pub fn k(&self) -> usize { unsafe { sys::yscv_cuda_i8b_k(self.raw) } }
    pub fn n(&self) -> usize { unsafe { sys::yscv_cuda_i8b_n(self.raw) } }
    /// b_zero_point of MatMulInteger / QLinearMatMul (scalar, runner/linear.rs:440-446).
    pub fn set_zero_point(&mut self, b_zero_point: i32) -> Result<(), CudaError> {
        check(unsafe { sys::yscv_cuda_i8b_set_zero_point(self.raw, b_zero_point) })
    }
    pub fn raw(&self) -> *const sys::yscv_cuda_i8b { self.raw }
}
impl Drop for PackedI8B {
    fn drop(&mut self) {
        if self.owned {
            // SAFETY: created by the library, freed once.
            unsafe { sys::yscv_cuda_i8b_free(self.raw) }
        }
    }
}

/// `pack_i8_b_for_matmul` (int8_matmul.rs:163-191).
pub fn pack_i8_b_for_matmul(b: &[i8], k: usize, n: usize) -> PackedI8B {
    debug_assert_eq!(b.len(), k * n);
    with_ctx(|ctx| {
        let mut raw = ptr::null_mut();
        // SAFETY: length checked above; the call synchronises before returning.
        check(unsafe { sys::yscv_cuda_pack_i8_b_for_matmul(ctx.raw(), b.as_ptr(), k, n, &mut raw) }).expect("pack_i8_b");
        PackedI8B { raw, owned: true }
    })
}

/// `int8_matmul_prepacked_dispatch` (int8_matmul.rs:2420-2425).
pub fn int8_matmul_prepacked_dispatch(a: &[i8], b: &PackedI8B, m: usize, out: &mut [i32]) {
    debug_assert_eq!(a.len(), m * b.k());
    debug_assert_eq!(out.len(), m * b.n());
    with_ctx(|ctx| {
        // SAFETY: lengths checked above.
        check(unsafe { sys::yscv_cuda_int8_matmul_prepacked(ctx.raw(), a.as_ptr(), b.raw, m, out.as_mut_ptr()) })
            .expect("int8_matmul_prepacked")
    })
}

/// `requant_i32_row_to_i8_dispatch` (int8_requant.rs:81-138).
pub fn requant_i32_row_to_i8_dispatch(acc: &[i32], bias: Option<&[i32]>, composite: f32, y_zp: f32, relu: bool,
                                      out: &mut [i8], c: usize) {
    debug_assert_eq!(acc.len(), out.len());
    debug_assert!(c > 0 && acc.len() % c == 0);
    if let Some(b) = bias {
        debug_assert_eq!(b.len(), c);
    }
    with_ctx(|ctx| {
        // SAFETY: lengths checked above.
        check(unsafe {
            sys::yscv_cuda_requant_i32_row_to_i8(ctx.raw(), acc.as_ptr(), bias.map_or(ptr::null(), |b| b.as_ptr()),
                                                 composite, y_zp, relu as c_int, out.as_mut_ptr(), acc.len(), c)
        })
        .expect("requant_i32_row_to_i8")
    })
}

/// How `exec_qlinear_matmul` rounds: the kernel-level contract (round half to even,
/// int8_requant.rs:143-169) or the runner's `f32::round` (runner/linear.rs:481-485).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum Rounding {
    TiesToEven,
    HalfAwayFromZero,
}

/// QLinearMatMul on a prepacked weight: `a` holds m x k bytes (uint8 when `a_unsigned`),
/// `out` m x n bytes in [qmin, qmax]. Any a_zero_point is exact.
#[allow(clippy::too_many_arguments)]
pub fn qlinear_matmul(ctx: &mut Context, a: &[u8], a_unsigned: bool, a_zero_point: i32, b: &PackedI8B, m: usize,
                      composite: f32, y_zero_point: f32, qmin: i32, qmax: i32, rounding: Rounding, out: &mut [u8])
                      -> Result<(), CudaError> {
    debug_assert_eq!(a.len(), m * b.k());
    debug_assert_eq!(out.len(), m * b.n());
    let rq = sys::yscv_cuda_requant {
        a_is_unsigned: a_unsigned as c_int,
        a_zero_point,
        composite,
        y_zero_point,
        qmin,
        qmax,
        round_mode: (rounding == Rounding::HalfAwayFromZero) as c_int,
    };
    // SAFETY: lengths checked above; `rq` lives across the synchronous call.
    check(unsafe { sys::yscv_cuda_qlinear_matmul(ctx.raw(), a.as_ptr().cast(), b.raw, m, &rq, out.as_mut_ptr().cast()) })
}

/// MatMulInteger on a prepacked weight: exact `(a - a_zero_point) x (b - b_zero_point)`.
pub fn matmul_integer(ctx: &mut Context, a: &[u8], a_unsigned: bool, a_zero_point: i32, b: &PackedI8B, m: usize,
                      out: &mut [i32]) -> Result<(), CudaError> {
    debug_assert_eq!(a.len(), m * b.k());
    debug_assert_eq!(out.len(), m * b.n());
    // SAFETY: lengths checked above.
    check(unsafe {
        sys::yscv_cuda_matmul_integer(ctx.raw(), a.as_ptr().cast(), a_unsigned as c_int, a_zero_point, b.raw, m,
                                      out.as_mut_ptr())
    })
}

// ---- the side tables, resident -----------------------------------------------------------------

/// `packed_int4_weights` / `prepacked_i8_weights` keyed by initializer name
/// (runner/linear.rs:228, plan/build.rs:1417-1454, runner/tensor_env.rs:178-183).
pub struct WeightRegistry(*mut sys::yscv_cuda_registry);
// SAFETY: the table is guarded by a reader-writer lock inside the library.
unsafe impl Send for WeightRegistry {}
unsafe impl Sync for WeightRegistry {}

/// Layout of an fp32 weight initializer as its node implies (packed_int4.rs:140-147).
#[derive(Clone, Copy, Debug)]
pub enum WeightLayout {
    MatMulKN = sys::YSCV_CUDA_WEIGHT_MATMUL_KN as isize,
    GemmNK = sys::YSCV_CUDA_WEIGHT_GEMM_NK as isize,
    GemmKN = sys::YSCV_CUDA_WEIGHT_GEMM_KN as isize,
}

impl WeightRegistry {
    pub fn new() -> Result<Self, CudaError> {
        let mut raw = ptr::null_mut();
        check(unsafe { sys::yscv_cuda_registry_create(&mut raw) })?;
        Ok(Self(raw))
    }

    /// One weight of `quantize_matmul_weights_int4_packed`; `Ok(false)` when the reference's
    /// rules skip it (k % group != 0, fewer than 32 weights) and the caller keeps the fp32 one.
    pub fn register_matmul_weight(&self, ctx: &mut Context, name: &str, weight: &[f32], dims: [usize; 2],
                                  layout: WeightLayout, group_size: usize) -> Result<bool, CudaError> {
        debug_assert_eq!(weight.len(), dims[0] * dims[1]);
        let cname = CString::new(name).expect("initializer names hold no NUL");
        let mut packed: c_int = 0;
        // SAFETY: length checked; the call synchronises before returning.
        check(unsafe {
            sys::yscv_cuda_registry_register_matmul_weight(ctx.raw(), self.0, cname.as_ptr(), weight.as_ptr(), dims[0],
                                                           dims[1], layout as c_int, group_size, &mut packed)
        })?;
        Ok(packed != 0)
    }

    /// The load-time prepack of a QLinearMatMul / MatMulInteger weight [k, n], behind
    /// `should_prepack_i8_b`.
    pub fn register_i8_weight(&self, ctx: &mut Context, name: &str, b: &[i8], k: usize, n: usize) -> Result<bool, CudaError> {
        debug_assert_eq!(b.len(), k * n);
        let cname = CString::new(name).expect("initializer names hold no NUL");
        let mut done: c_int = 0;
        check(unsafe { sys::yscv_cuda_registry_register_i8_weight(ctx.raw(), self.0, cname.as_ptr(), b.as_ptr(), k, n, &mut done) })?;
        Ok(done != 0)
    }

    pub fn int4(&self, name: &str) -> Option<ResidentInt4Weight> {
        let cname = CString::new(name).ok()?;
        let raw = unsafe { sys::yscv_cuda_registry_get_int4(self.0, cname.as_ptr()) };
        // the table keeps ownership: the view must not free the handle
        (!raw.is_null()).then(|| ResidentInt4Weight { raw: raw.cast_mut(), owned: false })
    }

    pub fn i8b(&self, name: &str) -> Option<PackedI8B> {
        let cname = CString::new(name).ok()?;
        let raw = unsafe { sys::yscv_cuda_registry_get_i8b(self.0, cname.as_ptr()) };
        (!raw.is_null()).then(|| PackedI8B { raw: raw.cast_mut(), owned: false })
    }

    pub fn len(&self) -> usize { unsafe { sys::yscv_cuda_registry_len(self.0) } }
    pub fn is_empty(&self) -> bool { self.len() == 0 }
}

impl Drop for WeightRegistry {
    fn drop(&mut self) { unsafe { sys::yscv_cuda_registry_destroy(self.0) } }
}

/// Process-wide registry for callers that mirror the reference's global tables.
pub fn global_registry() -> &'static WeightRegistry {
    static REG: OnceLock<WeightRegistry> = OnceLock::new();
    REG.get_or_init(|| WeightRegistry::new().expect("registry"))
}
