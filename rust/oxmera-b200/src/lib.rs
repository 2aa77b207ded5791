//! NOT COMPILED IN THIS ENVIRONMENT (no Rust toolchain here).
//!
//! The B200 backend for oxmera: `impl Backend` over the C ABI of
//! `liboxmera_b200.so` (hand-written sm_100a kernels).  One instance serves one
//! `Device::Cuda { index }`.
//!
//! It relies on four additions to the existing crates (the seam is not purely
//! additive):
//!
//! * `oxmera_core::DType::{BF16, F16, F8E4M3, F8E5M2}` (dtype.rs:9-22, the enum
//!   is `#[non_exhaustive]`); C tags 6, 7, 8, 9.
//! * `oxmera_core::Error::DivisionByZero { op }` (error.rs; `#[non_exhaustive]`),
//!   the "typed error" `BinaryOps::div` promises for integers (ops/lib.rs:47-49).
//! * A device variant of `StorageData` (storage.rs:24-32) with the two
//!   constructors used below:
//!   `Storage::device(ptr: NonNull<c_void>, bytes: usize, dtype, device, free: Box<dyn FnOnce(*mut c_void) + Send + Sync>)`
//!   and the accessor `Storage::device_ptr(&self) -> Option<NonNull<c_void>>`;
//!   `cpu_bytes()` keeps returning `None` for it (storage.rs:59-67).
//! * `MatmulOps::batched_matmul` (ops/lib.rs:53-59) with a default body that
//!   returns `NotImplemented`.
//!
//! Every operation allocates its output fresh and contiguous on this device
//! (ops/lib.rs:16-17), hands the three views to the library, and turns a
//! non-zero status into the `Error` variant with the same number.

pub mod ffi;

use std::ffi::{c_void, CStr};
use std::os::raw::c_int;
use std::ptr::NonNull;
use std::sync::Arc;

use oxmera_core::error::Error;
use oxmera_core::shape::broadcast_shapes;
use oxmera_core::{DType, Device, Layout, Result, Shape};
use oxmera_ops::{BinaryOps, MatmulOps, ReduceOps, UnaryOps};
use oxmera_runtime::Backend;
use oxmera_tensor::{Storage, Tensor};

/// The context handle, shared with the storages it allocated so that they can
/// free themselves after the backend value is gone.
struct Ctx(*mut ffi::oxm_ctx);
// The library serialises launches per context and may be called from any thread
// (`Backend: Send + Sync`, runtime/lib.rs:29).
unsafe impl Send for Ctx {}
unsafe impl Sync for Ctx {}
impl Drop for Ctx {
    fn drop(&mut self) {
        unsafe { ffi::oxm_ctx_destroy(self.0) };
    }
}

/// oxmera's B200 backend.
pub struct B200Backend {
    ctx: Arc<Ctx>,
    index: usize,
}

fn last_error() -> String {
    unsafe { CStr::from_ptr(ffi::oxm_last_error()) }.to_string_lossy().into_owned()
}

fn dtype_tag(dtype: DType) -> i32 {
    match dtype {
        DType::F32 => ffi::OXM_F32,
        DType::F64 => ffi::OXM_F64,
        DType::I32 => ffi::OXM_I32,
        DType::I64 => ffi::OXM_I64,
        DType::U8 => ffi::OXM_U8,
        DType::Bool => ffi::OXM_BOOL,
        DType::BF16 => ffi::OXM_BF16,
        DType::F16 => ffi::OXM_F16,
        DType::F8E4M3 => ffi::OXM_F8E4M3,
        DType::F8E5M2 => ffi::OXM_F8E5M2,
        _ => -1, // a dtype newer than this crate: the library answers UnsupportedDType
    }
}

impl B200Backend {
    /// The backend for `Device::Cuda { index }`.  `BackendUnavailable` when no
    /// sm_100 device with that index is visible (runtime/lib.rs:36-44).
    pub fn new(index: usize) -> Result<Self> {
        let mut ctx = std::ptr::null_mut();
        let st = unsafe { ffi::oxm_ctx_create(index as c_int, &mut ctx) };
        if st != ffi::OXM_OK {
            return Err(Self::error(st, "ctx_create", None, None, index));
        }
        Ok(Self { ctx: Arc::new(Ctx(ctx)), index })
    }

    fn raw(&self) -> *mut ffi::oxm_ctx {
        self.ctx.0
    }

    /// Status code -> the `Error` variant with the same number (error.rs:12-102).
    /// CUDA errors, expired device waits and bad arguments have no variant of
    /// their own and fold into `NotImplemented { op, detail }` with the
    /// library's message as the detail.
    fn error(st: c_int, op: &'static str, lhs: Option<&Tensor>, rhs: Option<&Tensor>, index: usize) -> Error {
        let shape_of = |t: Option<&Tensor>| t.map(|t| t.shape().clone()).unwrap_or_else(|| Shape::new(vec![]));
        let here = Device::Cuda { index };
        match st {
            ffi::OXM_SHAPE_MISMATCH => Error::ShapeMismatch { expected: shape_of(lhs), got: shape_of(rhs), op },
            ffi::OXM_BROADCAST_INCOMPATIBLE => Error::BroadcastIncompatible { lhs: shape_of(lhs), rhs: shape_of(rhs) },
            ffi::OXM_DTYPE_MISMATCH => Error::DTypeMismatch {
                expected: lhs.map(|t| t.dtype()).unwrap_or(DType::F32),
                got: rhs.map(|t| t.dtype()).unwrap_or(DType::F32),
                op,
            },
            ffi::OXM_UNSUPPORTED_DTYPE => Error::UnsupportedDType { dtype: lhs.map(|t| t.dtype()).unwrap_or(DType::F32), op },
            ffi::OXM_DEVICE_MISMATCH => Error::DeviceMismatch {
                lhs: lhs.map(|t| t.device()).unwrap_or(here),
                rhs: rhs.map(|t| t.device()).unwrap_or(here),
                op,
            },
            ffi::OXM_INDEX_OUT_OF_BOUNDS => Error::IndexOutOfBounds { index: vec![], shape: shape_of(lhs) },
            ffi::OXM_BACKEND_UNAVAILABLE => Error::BackendUnavailable { device: here },
            ffi::OXM_DIVIDE_BY_ZERO => Error::DivisionByZero { op },
            _ => Error::NotImplemented { op, detail: last_error() },
        }
    }

    fn fail(&self, st: c_int, op: &'static str, lhs: Option<&Tensor>, rhs: Option<&Tensor>) -> Error {
        Self::error(st, op, lhs, rhs, self.index)
    }

    /// The view the library sees: the tensor's layout plus its storage pointer.
    fn view(&self, t: &Tensor, op: &'static str) -> Result<ffi::oxm_view> {
        let layout = t.layout();
        let dims = layout.shape.dims();
        if dims.len() > ffi::OXM_MAX_DIMS {
            return Err(Error::NotImplemented { op, detail: format!("rank {}", dims.len()) });
        }
        if t.device() != self.device() {
            return Err(Error::DeviceMismatch { lhs: t.device(), rhs: self.device(), op });
        }
        let mut v = ffi::oxm_view {
            dtype: dtype_tag(t.dtype()),
            ndim: dims.len() as i32,
            shape: [0; ffi::OXM_MAX_DIMS],
            strides: [0; ffi::OXM_MAX_DIMS],
            offset: layout.offset as i64,
            base: t.storage().device_ptr().map(|p| p.as_ptr()).unwrap_or(std::ptr::null_mut()),
            device: self.index as i32,
            reserved: 0,
        };
        for (i, (&d, &s)) in dims.iter().zip(layout.strides.values()).enumerate() {
            v.shape[i] = d as i64;
            v.strides[i] = s as i64;
        }
        Ok(v)
    }

    /// A fresh contiguous tensor on this device (ops/lib.rs:16-17).  Allocation is
    /// stream-ordered and pooled; the storage frees itself through the context.
    pub fn empty(&self, shape: Shape, dtype: DType) -> Result<Tensor> {
        let bytes = shape.numel() * dtype.size_in_bytes();
        let mut ptr: *mut c_void = std::ptr::null_mut();
        let st = unsafe { ffi::oxm_alloc(self.raw(), bytes, &mut ptr) };
        if st != ffi::OXM_OK {
            return Err(self.fail(st, "alloc", None, None));
        }
        let ctx = Arc::clone(&self.ctx);
        let storage = Storage::device(
            NonNull::new(ptr).expect("oxm_alloc returned null with OXM_OK"),
            bytes,
            dtype,
            self.device(),
            Box::new(move |p| {
                unsafe { ffi::oxm_free(ctx.0, p) };
            }),
        );
        Tensor::from_storage(Arc::new(storage), Layout::contiguous(shape))
    }

    /// A contiguous device tensor holding `bytes` (host memory, `dtype` encoding).
    /// Stands in for `Tensor::from_vec_f32` (tensor.rs:29-36), which is CPU-f32 only.
    pub fn from_host_bytes(&self, bytes: &[u8], dtype: DType, shape: Shape) -> Result<Tensor> {
        if bytes.len() != shape.numel() * dtype.size_in_bytes() {
            return Err(Error::ShapeMismatch { expected: shape.clone(), got: Shape::new(vec![bytes.len() / dtype.size_in_bytes()]), op: "from_host_bytes" });
        }
        let t = self.empty(shape, dtype)?;
        let dst = t.storage().device_ptr().map(|p| p.as_ptr()).unwrap_or(std::ptr::null_mut());
        let st = unsafe { ffi::oxm_h2d(self.raw(), dst, bytes.as_ptr().cast(), bytes.len()) };
        if st != ffi::OXM_OK {
            return Err(self.fail(st, "from_host_bytes", None, None));
        }
        // the source slice may be pageable: wait until the copy has consumed it
        self.synchronize()?;
        Ok(t)
    }

    /// The elements of `t` in logical order, as host bytes.  Returns after the
    /// bytes have landed and reports any pending device-side failure.
    pub fn to_host_bytes(&self, t: &Tensor) -> Result<Vec<u8>> {
        let c = if t.layout().is_contiguous() { t.clone() } else { self.contiguous(t)? };
        let esz = c.dtype().size_in_bytes();
        let mut out = vec![0u8; c.shape().numel() * esz];
        let base = c.storage().device_ptr().map(|p| p.as_ptr()).unwrap_or(std::ptr::null_mut());
        let src = unsafe { base.cast::<u8>().add(c.layout().offset * esz) };
        let st = unsafe { ffi::oxm_d2h(self.raw(), out.as_mut_ptr().cast(), src.cast(), out.len()) };
        if st != ffi::OXM_OK {
            return Err(self.fail(st, "to_host_bytes", Some(t), None));
        }
        Ok(out)
    }

    /// The device half of `Tensor::contiguous` (tensor.rs:86-90).
    pub fn contiguous(&self, t: &Tensor) -> Result<Tensor> {
        let out = self.empty(t.shape().clone(), t.dtype())?;
        let (s, d) = (self.view(t, "contiguous")?, self.view(&out, "contiguous")?);
        let st = unsafe { ffi::oxm_contiguous(self.raw(), &s, &d) };
        if st != ffi::OXM_OK {
            return Err(self.fail(st, "contiguous", Some(t), Some(&out)));
        }
        Ok(out)
    }

    /// Wait for everything submitted so far; surfaces device-side failures.
    pub fn synchronize(&self) -> Result<()> {
        match unsafe { ffi::oxm_sync(self.raw()) } {
            ffi::OXM_OK => Ok(()),
            st => Err(self.fail(st, "sync", None, None)),
        }
    }

    fn matmul_with(&self, lhs: &Tensor, rhs: &Tensor, batched: bool) -> Result<Tensor> {
        let op: &'static str = if batched { "batched_matmul" } else { "matmul" };
        let (a, b) = (self.view(lhs, op)?, self.view(rhs, op)?);
        let (ld, rd) = (lhs.shape().dims(), rhs.shape().dims());
        // Enough of the output shape to allocate it; the library validates and reports the typed error.
        let out_shape = if ld.len() >= 2 && rd.len() >= 2 && (batched || (ld.len() == 2 && rd.len() == 2)) {
            let lead = broadcast_shapes(&Shape::new(ld[..ld.len() - 2].to_vec()), &Shape::new(rd[..rd.len() - 2].to_vec()))?;
            let mut dims = lead.dims().to_vec();
            dims.push(ld[ld.len() - 2]);
            dims.push(rd[rd.len() - 1]);
            Shape::new(dims)
        } else {
            Shape::new(vec![1, 1]) // the library refuses these ranks
        };
        let out = self.empty(out_shape, lhs.dtype())?;
        let o = self.view(&out, op)?;
        let st = unsafe {
            if batched { ffi::oxm_batched_matmul(self.raw(), &a, &b, &o) } else { ffi::oxm_matmul(self.raw(), &a, &b, &o) }
        };
        if st != ffi::OXM_OK {
            return Err(self.fail(st, op, Some(lhs), Some(rhs)));
        }
        Ok(out)
    }

    /// The block-scaled fp8 product (MXFP8): `lhs_scale` `[.., M, K/32]` and
    /// `rhs_scale` `[.., K/32, N]` are U8 tensors of E8M0 exponents, one per 32
    /// contraction elements of every row of `lhs` and column of `rhs`.
    pub fn matmul_mx(&self, lhs: &Tensor, lhs_scale: &Tensor, rhs: &Tensor, rhs_scale: &Tensor, out_dtype: DType) -> Result<Tensor> {
        let op = "matmul_mx";
        let (a, b) = (self.view(lhs, op)?, self.view(rhs, op)?);
        let (sa, sb) = (self.view(lhs_scale, op)?, self.view(rhs_scale, op)?);
        let (ld, rd) = (lhs.shape().dims(), rhs.shape().dims());
        if ld.len() < 2 || rd.len() < 2 {
            return Err(Error::ShapeMismatch { expected: lhs.shape().clone(), got: rhs.shape().clone(), op });
        }
        let lead = broadcast_shapes(&Shape::new(ld[..ld.len() - 2].to_vec()), &Shape::new(rd[..rd.len() - 2].to_vec()))?;
        let mut dims = lead.dims().to_vec();
        dims.push(ld[ld.len() - 2]);
        dims.push(rd[rd.len() - 1]);
        let out = self.empty(Shape::new(dims), out_dtype)?;
        let o = self.view(&out, op)?;
        let st = unsafe { ffi::oxm_matmul_mx(self.raw(), &a, &sa, &b, &sb, &o) };
        if st != ffi::OXM_OK {
            return Err(self.fail(st, op, Some(lhs), Some(rhs)));
        }
        Ok(out)
    }

    /// `act(lhs . rhs + bias)`, optionally added into `accumulate_into`
    /// (gradient accumulation), in one kernel.
    pub fn matmul_fused(&self, lhs: &Tensor, rhs: &Tensor, bias: Option<&Tensor>, activation: i32, accumulate_into: Option<&Tensor>) -> Result<Tensor> {
        let op = "matmul_fused";
        let (a, b) = (self.view(lhs, op)?, self.view(rhs, op)?);
        let out = match accumulate_into {
            Some(t) => t.clone(),
            None => {
                let (ld, rd) = (lhs.shape().dims(), rhs.shape().dims());
                if ld.len() < 2 || rd.len() < 2 {
                    return Err(Error::ShapeMismatch { expected: lhs.shape().clone(), got: rhs.shape().clone(), op });
                }
                let lead = broadcast_shapes(&Shape::new(ld[..ld.len() - 2].to_vec()), &Shape::new(rd[..rd.len() - 2].to_vec()))?;
                let mut dims = lead.dims().to_vec();
                dims.push(ld[ld.len() - 2]);
                dims.push(rd[rd.len() - 1]);
                self.empty(Shape::new(dims), lhs.dtype())?
            }
        };
        let o = self.view(&out, op)?;
        let bias_view = match bias {
            Some(t) => Some(self.view(t, op)?),
            None => None,
        };
        let ep = ffi::oxm_epilogue {
            bias: bias_view.as_ref().map(|v| v as *const _).unwrap_or(std::ptr::null()),
            activation,
            accumulate: accumulate_into.is_some() as i32,
        };
        let st = unsafe { ffi::oxm_matmul_fused(self.raw(), &a, &b, &o, &ep) };
        if st != ffi::OXM_OK {
            return Err(self.fail(st, op, Some(lhs), Some(rhs)));
        }
        Ok(out)
    }

    fn unary(&self, code: c_int, op: &'static str, a: &Tensor) -> Result<Tensor> {
        let va = self.view(a, op)?;
        let out = self.empty(a.shape().clone(), a.dtype())?;
        let vo = self.view(&out, op)?;
        match unsafe { ffi::oxm_unary(self.raw(), code, &va, &vo) } {
            ffi::OXM_OK => Ok(out),
            st => Err(self.fail(st, op, Some(a), None)),
        }
    }

    fn binary(&self, code: c_int, op: &'static str, lhs: &Tensor, rhs: &Tensor) -> Result<Tensor> {
        let (va, vb) = (self.view(lhs, op)?, self.view(rhs, op)?);
        let out = self.empty(broadcast_shapes(lhs.shape(), rhs.shape())?, lhs.dtype())?;
        let vo = self.view(&out, op)?;
        match unsafe { ffi::oxm_binary(self.raw(), code, &va, &vb, &vo) } {
            ffi::OXM_OK => Ok(out),
            st => Err(self.fail(st, op, Some(lhs), Some(rhs))),
        }
    }

    fn reduce(&self, code: c_int, op: &'static str, a: &Tensor, axes: &[usize]) -> Result<Tensor> {
        let va = self.view(a, op)?;
        let dims = a.shape().dims();
        if axes.iter().any(|&x| x >= dims.len()) {
            return Err(Error::IndexOutOfBounds { index: axes.to_vec(), shape: a.shape().clone() });
        }
        let kept: Vec<usize> = if axes.is_empty() {
            vec![]
        } else {
            dims.iter().enumerate().filter(|(d, _)| !axes.contains(d)).map(|(_, &s)| s).collect()
        };
        let out = self.empty(Shape::new(kept), a.dtype())?;
        let vo = self.view(&out, op)?;
        let ax: Vec<i32> = axes.iter().map(|&x| x as i32).collect();
        match unsafe { ffi::oxm_reduce(self.raw(), code, &va, ax.as_ptr(), ax.len() as c_int, &vo) } {
            ffi::OXM_OK => Ok(out),
            st => Err(self.fail(st, op, Some(a), None)),
        }
    }
}

impl UnaryOps for B200Backend {
    fn neg(&self, a: &Tensor) -> Result<Tensor> {
        self.unary(ffi::OXM_NEG, "neg", a)
    }
    fn exp(&self, a: &Tensor) -> Result<Tensor> {
        self.unary(ffi::OXM_EXP, "exp", a)
    }
    fn ln(&self, a: &Tensor) -> Result<Tensor> {
        self.unary(ffi::OXM_LN, "ln", a)
    }
    fn abs(&self, a: &Tensor) -> Result<Tensor> {
        self.unary(ffi::OXM_ABS, "abs", a)
    }
}

impl BinaryOps for B200Backend {
    fn add(&self, lhs: &Tensor, rhs: &Tensor) -> Result<Tensor> {
        self.binary(ffi::OXM_ADD, "add", lhs, rhs)
    }
    fn sub(&self, lhs: &Tensor, rhs: &Tensor) -> Result<Tensor> {
        self.binary(ffi::OXM_SUB, "sub", lhs, rhs)
    }
    fn mul(&self, lhs: &Tensor, rhs: &Tensor) -> Result<Tensor> {
        self.binary(ffi::OXM_MUL, "mul", lhs, rhs)
    }
    /// Integer division by zero comes back as `Error::DivisionByZero` from this
    /// call itself: the integer form waits for its kernel.
    fn div(&self, lhs: &Tensor, rhs: &Tensor) -> Result<Tensor> {
        self.binary(ffi::OXM_DIV, "div", lhs, rhs)
    }
}

impl MatmulOps for B200Backend {
    fn matmul(&self, lhs: &Tensor, rhs: &Tensor) -> Result<Tensor> {
        self.matmul_with(lhs, rhs, false)
    }
    fn batched_matmul(&self, lhs: &Tensor, rhs: &Tensor) -> Result<Tensor> {
        self.matmul_with(lhs, rhs, true)
    }
}

impl ReduceOps for B200Backend {
    fn sum(&self, a: &Tensor, axes: &[usize]) -> Result<Tensor> {
        self.reduce(ffi::OXM_SUM, "sum", a, axes)
    }
    fn max(&self, a: &Tensor, axes: &[usize]) -> Result<Tensor> {
        self.reduce(ffi::OXM_MAX, "max", a, axes)
    }
}

impl Backend for B200Backend {
    fn device(&self) -> Device {
        Device::Cuda { index: self.index }
    }
    fn name(&self) -> &'static str {
        "b200-tcgen05"
    }
}

/// Register the backend for `Device::Cuda { index }` (runtime/lib.rs:46-53:
/// "backend crates call this from their initialization").
pub fn register(index: usize) -> Result<()> {
    oxmera_runtime::register_backend(Arc::new(B200Backend::new(index)?));
    Ok(())
}

/// Register one backend per visible sm_100 device; returns how many.
pub fn register_all() -> Result<usize> {
    let mut n: c_int = 0;
    unsafe { ffi::oxm_device_count(&mut n) };
    let mut registered = 0;
    for index in 0..n.max(0) as usize {
        match register(index) {
            Ok(()) => registered += 1,
            Err(Error::BackendUnavailable { .. }) => {} // another architecture in the same box
            Err(e) => return Err(e),
        }
    }
    Ok(registered)
}
