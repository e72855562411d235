//! `cubek_quant::{quantize, dequantize}::launch_ref` on B200, through the C ABI of
//! `libcubek_quant_b200.so` (declared in `include/cubek_quant_b200.h`).
//!
//! The reference entry points borrow `TensorHandleRef`s of a CubeCL runtime
//! (crates/cubek-quant/src/quantize.rs:174-182, crates/cubek-quant/src/dequantize.rs:171-178).
//! This shim keeps their argument order and their error behaviour (panic where the reference
//! panics, `Err` where it returns `Err`) over a minimal handle type that carries what the reference
//! reads from a handle: device pointer, shape, strides, element size.
//!
//! Not compiled where this repository is built (no Rust toolchain there).

use core::ffi::{c_char, c_int, c_void};
use std::ffi::CStr;

// ---- scheme (mirrors `cubecl_common::quant::scheme`, re-exported at crates/cubek-quant/src/lib.rs:14) ----

#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum ElemType { F32 = 0, F16 = 1, BF16 = 2 }

#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum QuantValue { Q8F = 0, Q8S = 1, Q4F = 2, Q4S = 3, Q2F = 4, Q2S = 5, E4M3 = 6, E5M2 = 7, E2M1 = 8 }

#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum QuantStore { Native = 0, U32 = 1 }

#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum QuantParam { F32 = 0, F16 = 1, BF16 = 2 }

#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum QuantMode { Symmetric = 0 }

/// Block extents are `u8`, as in the reference (`QuantLevel::block([b as u8])`, symmetric.rs:202).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum QuantLevel { Tensor, Block { rank: u8, dims: [u8; 8] } }

impl QuantLevel {
    pub fn block(dims: &[u8]) -> Self {
        assert!(!dims.is_empty() && dims.len() <= 8, "a block size has 1 to 8 dims");
        let mut d = [0u8; 8];
        d[..dims.len()].copy_from_slice(dims);
        QuantLevel::Block { rank: dims.len() as u8, dims: d }
    }
}

#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub struct QuantScheme {
    pub value: QuantValue,
    pub param: QuantParam,
    pub store: QuantStore,
    pub level: QuantLevel,
    pub mode: QuantMode,
}

impl Default for QuantScheme {
    fn default() -> Self {
        Self { value: QuantValue::Q8F, param: QuantParam::F32, store: QuantStore::U32, level: QuantLevel::Tensor, mode: QuantMode::Symmetric }
    }
}

impl QuantScheme {
    pub fn with_level(mut self, level: QuantLevel) -> Self { self.level = level; self }
    pub fn with_mode(mut self, mode: QuantMode) -> Self { self.mode = mode; self }
    pub fn with_value(mut self, value: QuantValue) -> Self { self.value = value; self }
    pub fn with_store(mut self, store: QuantStore) -> Self { self.store = store; self }
    pub fn with_param(mut self, param: QuantParam) -> Self { self.param = param; self }

    /// Quantized values per stored item (quantize.rs:144, :290).
    pub fn num_quants(&self) -> usize {
        unsafe { qk_num_quants(&self.to_c()) as usize }
    }

    fn to_c(&self) -> QkScheme {
        let (level, block_rank, block) = match self.level {
            QuantLevel::Tensor => (0, 0, [0u8; 8]),
            QuantLevel::Block { rank, dims } => (1, rank as i32, dims),
        };
        QkScheme { value: self.value as i32, param: self.param as i32, store: self.store as i32, level, mode: self.mode as i32, block_rank, block }
    }
}

// ---- handles ----

/// What the reference reads from a `TensorHandleRef` (layout/scales.rs:213-215, quantize.rs:234-239):
/// the device buffer, shape, strides (in elements) and element size.
#[derive(Clone, Copy, Debug)]
pub struct TensorHandleRef<'a> {
    pub ptr: *mut c_void,
    pub shape: &'a [usize],
    pub strides: &'a [usize],
    pub elem_size: usize,
}

/// Stands in for `ComputeClient`: the CUDA stream launches are enqueued on (the current device is used).
#[derive(Clone, Copy, Debug)]
pub struct ComputeClient { pub stream: *mut c_void }

#[derive(Debug)]
pub enum LaunchError { Layout(String), Align(String), Workspace(String), Cuda(String), Other(String) }

// ---- raw ABI ----

#[repr(C)]
struct QkScheme { value: i32, param: i32, store: i32, level: i32, mode: i32, block_rank: i32, block: [u8; 8] }

#[repr(C)]
struct QkTensor { ptr: *mut c_void, rank: i32, shape: *const i64, strides: *const i64, elem_size: i32 }

extern "C" {
    fn qk_num_quants(scheme: *const QkScheme) -> c_int;
    fn qk_quantize(input: *const QkTensor, output: *const QkTensor, scale: *const QkTensor, out_scale: *const QkTensor,
                   scheme: *const QkScheme, input_dtype: c_int, stream: *mut c_void) -> c_int;
    fn qk_dequantize(values: *const QkTensor, output: *const QkTensor, params: *const QkTensor,
                     scheme: *const QkScheme, output_dtype: c_int, stream: *mut c_void) -> c_int;
    fn qk_compute_scales(input: *const QkTensor, scale: *const QkTensor, scheme: *const QkScheme, input_dtype: c_int,
                         workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    fn qk_quantize_dynamic(input: *const QkTensor, output: *const QkTensor, out_scale: *const QkTensor,
                           scheme: *const QkScheme, input_dtype: c_int, workspace: *mut c_void, workspace_bytes: usize,
                           stream: *mut c_void) -> c_int;
    fn qk_workspace_bytes() -> usize;
    fn qk_strerror(status: c_int) -> *const c_char;
}

struct Marshalled { shape: Vec<i64>, strides: Vec<i64>, ptr: *mut c_void, elem_size: i32 }

impl Marshalled {
    fn new(h: &TensorHandleRef<'_>) -> Self {
        Self {
            shape: h.shape.iter().map(|&s| s as i64).collect(),
            strides: h.strides.iter().map(|&s| s as i64).collect(),
            ptr: h.ptr,
            elem_size: h.elem_size as i32,
        }
    }
    fn as_c(&self) -> QkTensor {
        QkTensor { ptr: self.ptr, rank: self.shape.len() as i32, shape: self.shape.as_ptr(), strides: self.strides.as_ptr(), elem_size: self.elem_size }
    }
}

fn message(status: c_int) -> String {
    unsafe { CStr::from_ptr(qk_strerror(status)).to_string_lossy().into_owned() }
}

/// Status codes 1..=4 are the reference's `panic!` / `assert!` sites (quantize.rs:203-206, :218, :273, :324;
/// dequantize.rs:205-208, :226, :278, :330; lib.rs:28-31); the others are launch errors.
fn finish(status: c_int) -> Result<(), LaunchError> {
    match status {
        0 => Ok(()),
        1..=4 => panic!("{}", message(status)),
        5 => Err(LaunchError::Layout(message(status))),
        6 => Err(LaunchError::Align(message(status))),
        8 => Err(LaunchError::Workspace(message(status))),
        s if s >= 1000 => Err(LaunchError::Cuda(message(status))),
        _ => Err(LaunchError::Other(message(status))),
    }
}

pub mod quantize {
    use super::*;

    /// `cubek_quant::quantize::launch_ref` (quantize.rs:174-221): same arguments, same order.
    pub fn launch_ref(client: &ComputeClient, input: &TensorHandleRef<'_>, output: &TensorHandleRef<'_>,
                      scale: &TensorHandleRef<'_>, out_scale: &TensorHandleRef<'_>, scheme: &QuantScheme,
                      input_elem: ElemType) -> Result<(), LaunchError> {
        let (i, o, s, os) = (Marshalled::new(input), Marshalled::new(output), Marshalled::new(scale), Marshalled::new(out_scale));
        finish(unsafe {
            qk_quantize(&i.as_c(), &o.as_c(), &s.as_c(), &os.as_c(), &scheme.to_c(), input_elem as c_int, client.stream)
        })
    }

    /// The caller-side absmax + scale formula (`cubek_reduce` MaxAbs, then `2*absmax/(q_max-q_min)`).
    pub fn compute_scales(client: &ComputeClient, input: &TensorHandleRef<'_>, scale: &TensorHandleRef<'_>,
                          scheme: &QuantScheme, input_elem: ElemType, workspace: *mut c_void, workspace_bytes: usize)
                          -> Result<(), LaunchError> {
        let (i, s) = (Marshalled::new(input), Marshalled::new(scale));
        finish(unsafe {
            qk_compute_scales(&i.as_c(), &s.as_c(), &scheme.to_c(), input_elem as c_int, workspace, workspace_bytes, client.stream)
        })
    }

    /// compute_scales + launch_ref fused, identical results.
    pub fn launch_dynamic(client: &ComputeClient, input: &TensorHandleRef<'_>, output: &TensorHandleRef<'_>,
                          out_scale: &TensorHandleRef<'_>, scheme: &QuantScheme, input_elem: ElemType,
                          workspace: *mut c_void, workspace_bytes: usize) -> Result<(), LaunchError> {
        let (i, o, os) = (Marshalled::new(input), Marshalled::new(output), Marshalled::new(out_scale));
        finish(unsafe {
            qk_quantize_dynamic(&i.as_c(), &o.as_c(), &os.as_c(), &scheme.to_c(), input_elem as c_int, workspace,
                                workspace_bytes, client.stream)
        })
    }

    pub fn workspace_bytes() -> usize { unsafe { qk_workspace_bytes() } }
}

pub mod dequantize {
    use super::*;

    /// `cubek_quant::dequantize::launch_ref` (dequantize.rs:171-229): same arguments, same order.
    pub fn launch_ref(client: &ComputeClient, values: &TensorHandleRef<'_>, output: &TensorHandleRef<'_>,
                      params: &TensorHandleRef<'_>, scheme: &QuantScheme, input_dtype: ElemType)
                      -> Result<(), LaunchError> {
        let (v, o, p) = (Marshalled::new(values), Marshalled::new(output), Marshalled::new(params));
        finish(unsafe { qk_dequantize(&v.as_c(), &o.as_c(), &p.as_c(), &scheme.to_c(), input_dtype as c_int, client.stream) })
    }
}
