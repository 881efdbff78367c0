//! UNVERIFIED: no rustc in the image this repository is built in; never compiled.
//!
//! `CudaBackend`: yaxus's `Backend` (crates/yaxus-model/src/lib.rs:95-171) and `SyncReadback`
//! (:177-185) over libyaxus_cuda, for NVIDIA B200 (sm_100a).
//!
//! Every method is a thin call into the C ABI (`ffi.rs`), with the error behaviour the trait
//! prescribes: the operators cannot fail by signature, so the library keeps the first error and
//! the next read-back reports it, which is where the reference surfaces a lost device too
//! (crates/yaxus-model/src/lib.rs:187-197).  Weights are taken as bf16 (`Quant::Bf16`); the
//! reference's quantised formats are refused at load.
//!
//! The page tables, the page allocator and prefix sharing stay in yaxus-model
//! (crates/yaxus-model/src/kv.rs); they reach the library only as `PassMeta` arrays and
//! `copy_page` calls, unchanged.
mod ffi;

use std::ffi::CStr;
use std::os::raw::c_void;
use std::sync::{Arc, Mutex};

use anyhow::{anyhow, bail, Result};
use yaxus_model::{Backend, Config, LayerMeta, PassMeta, Quant, SyncReadback, TensorRef};

/// One device context, shared by the target and the draft model the way `GpuBackend::share`
/// shares a device (crates/yaxus-backend-gpu/src/lib.rs:235-246).  A context is driven by one
/// thread at a time (the engine's inference thread, docs/DESIGN.md:131): hence the mutex.
struct Ctx(*mut ffi::yx_ctx);
unsafe impl Send for Ctx {}
impl Drop for Ctx {
    fn drop(&mut self) {
        unsafe { ffi::yx_ctx_destroy(self.0) }
    }
}

/// A row-major `[rows, cols]` f32 activation in device memory.
pub struct Tensor {
    ptr: *mut c_void,
    pub rows: usize,
    pub cols: usize,
    ctx: Arc<Mutex<Ctx>>,
}
unsafe impl Send for Tensor {}
impl Drop for Tensor {
    fn drop(&mut self) {
        // Stream-ordered with the kernels that still read it: cudaFree waits for the device.
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_tensor_free(ctx.0, self.ptr) };
    }
}

/// A weight in device memory.  Norm vectors are held as f32, like the GPU backend's
/// `Weight::Vector` (crates/yaxus-backend-gpu/src/weights.rs:290-294).
pub struct Weight {
    ptr: *mut c_void,
    pub shape: Vec<usize>,
    bytes: usize,
    ctx: Arc<Mutex<Ctx>>,
}
unsafe impl Send for Weight {}
impl Drop for Weight {
    fn drop(&mut self) {
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_tensor_free(ctx.0, self.ptr) };
    }
}

/// Paged K/V storage of all layers of one model.  Opaque to yaxus-model; the physical layout
/// is the library's, the slot semantics (`page * 128 + pos % 128`) are the reference's.
pub struct Kv {
    ptr: *mut ffi::yx_kv,
    ctx: Arc<Mutex<Ctx>>,
}
unsafe impl Send for Kv {}
impl Drop for Kv {
    fn drop(&mut self) {
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_kv_destroy(ctx.0, self.ptr) };
    }
}

/// Storage type of the KV cache.  `F32` is the reference's; the 16-bit types round on append
/// (round to nearest even) and halve the bytes the decode kernels stream.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum KvDtype {
    F32,
    F16,
    Bf16,
}

pub struct CudaBackend {
    ctx: Arc<Mutex<Ctx>>,
    device: i32,
    kv_dtype: KvDtype,
    /// Rows and token ids of the current pass (`embed` gathers by id).
    rows: usize,
    ids: Vec<u32>,
    weight_bytes: usize,
}

fn last_error(ctx: &Ctx) -> String {
    unsafe { CStr::from_ptr(ffi::yx_last_error(ctx.0)).to_string_lossy().into_owned() }
}

impl CudaBackend {
    /// A backend on CUDA device `device`.  Fails when there is no sm_100 device: the library
    /// has no CPU fallback.
    pub fn new(device: i32) -> Result<Self> {
        let mut raw = std::ptr::null_mut();
        let rc = unsafe { ffi::yx_ctx_create(device, std::ptr::null_mut(), &mut raw) };
        if rc != ffi::YX_OK {
            bail!("yx_ctx_create({device}) failed with code {rc}: no usable CUDA device (sm_100a is required)");
        }
        Ok(CudaBackend { ctx: Arc::new(Mutex::new(Ctx(raw))), device, kv_dtype: KvDtype::F16, rows: 0, ids: Vec::new(), weight_bytes: 0 })
    }

    /// A second backend on the same device context, for the draft model.
    pub fn share_for_draft(&self) -> Self {
        CudaBackend { ctx: self.ctx.clone(), device: self.device, kv_dtype: self.kv_dtype, rows: 0, ids: Vec::new(), weight_bytes: 0 }
    }

    pub fn set_kv_dtype(&mut self, dtype: KvDtype) {
        self.kv_dtype = dtype;
    }

    fn alloc(&self, rows: usize, cols: usize) -> Tensor {
        let mut ptr = std::ptr::null_mut();
        let ctx = self.ctx.lock().unwrap();
        // A failed allocation sticks to the context like any other error; the tensor is then
        // null and every later call is refused until the read-back reports it.
        unsafe { ffi::yx_tensor_alloc(ctx.0, rows * cols * 4, &mut ptr) };
        drop(ctx);
        Tensor { ptr, rows, cols, ctx: self.ctx.clone() }
    }

    /// The sticky error, if any, as the read-back's `Err`.
    fn check(&self) -> Result<()> {
        let ctx = self.ctx.lock().unwrap();
        let rc = unsafe { ffi::yx_sync(ctx.0) };
        if rc != ffi::YX_OK {
            let msg = last_error(&ctx);
            unsafe { ffi::yx_clear_error(ctx.0) };
            return Err(anyhow!("CUDA backend error {rc}: {msg}"));
        }
        Ok(())
    }
}

impl Backend for CudaBackend {
    type Tensor = Tensor;
    type Weight = Weight;
    type Kv = Kv;

    fn name(&self) -> String {
        format!("cuda:{} (sm_100a)", self.device)
    }

    fn weight_bytes(&self) -> usize {
        self.weight_bytes
    }

    /// Vectors are uploaded as f32 (the library's norm entries take f32, like the GPU backend's
    /// `Weight::Vector`); matrices and the embedding table as the bf16 the file holds
    /// (cpu lib.rs:455-462).  Quantised formats are the reference's other backends' business.
    fn load_weight(&mut self, t: &TensorRef, quant: Quant) -> Result<Weight> {
        if t.shape.len() != 1 && !matches!(quant, Quant::Bf16) {
            bail!("the CUDA backend takes bf16 weights only (asked for {quant:?})");
        }
        let host: Vec<u8> = if t.shape.len() == 1 {
            t.to_f32_vec()?.iter().flat_map(|v| v.to_le_bytes()).collect()
        } else {
            t.to_bf16_vec().iter().flat_map(|v| v.to_le_bytes()).collect()
        };
        let bytes = host.len();
        let mut ptr = std::ptr::null_mut();
        let ctx = self.ctx.lock().unwrap();
        let rc = unsafe { ffi::yx_tensor_alloc(ctx.0, bytes, &mut ptr) };
        if rc != ffi::YX_OK {
            bail!("load_weight: {}", last_error(&ctx));
        }
        // Pageable source: the library copies it into its pinned ring before the call returns.
        let rc = unsafe { ffi::yx_upload(ctx.0, ptr, host.as_ptr() as *const c_void, bytes) };
        if rc != ffi::YX_OK || unsafe { ffi::yx_sync(ctx.0) } != ffi::YX_OK {
            bail!("load_weight: {}", last_error(&ctx));
        }
        drop(ctx);
        self.weight_bytes += bytes;
        Ok(Weight { ptr, shape: t.shape.clone(), bytes, ctx: self.ctx.clone() })
    }

    /// crates/yaxus-model/src/lib.rs:118.  Zeroed arenas for every layer; each layer's window
    /// and RoPE parameters travel with the storage.
    fn new_kv(&mut self, cfg: &Config, metas: &[LayerMeta], pages: usize, max_pos: usize) -> Result<Kv> {
        let layers: Vec<ffi::yx_layer> = metas
            .iter()
            .map(|m| {
                let mut inv_freq = [0f32; ffi::YX_HEAD_DIM / 2];
                inv_freq[..m.rope.inv_freq.len().min(64)].copy_from_slice(&m.rope.inv_freq[..m.rope.inv_freq.len().min(64)]);
                ffi::yx_layer {
                    window: m.window.map(|w| w.min(i32::MAX as usize) as i32).unwrap_or(0),
                    rope: ffi::yx_rope { inv_freq, concentration: m.rope.concentration },
                }
            })
            .collect();
        let dtype = match self.kv_dtype {
            KvDtype::F32 => ffi::YX_F32,
            KvDtype::F16 => ffi::YX_F16,
            KvDtype::Bf16 => ffi::YX_BF16,
        };
        let mut kv = std::ptr::null_mut();
        let ctx = self.ctx.lock().unwrap();
        let rc = unsafe {
            ffi::yx_kv_create(
                ctx.0,
                layers.len() as i32,
                layers.as_ptr(),
                pages as u32,
                cfg.num_key_value_heads as i32,
                cfg.head_dim as i32,
                dtype,
                max_pos as u32,
                &mut kv,
            )
        };
        if rc != ffi::YX_OK {
            let msg = last_error(&ctx);
            unsafe { ffi::yx_clear_error(ctx.0) };
            bail!("new_kv: {msg}");
        }
        drop(ctx);
        Ok(Kv { ptr: kv, ctx: self.ctx.clone() })
    }

    /// crates/yaxus-model/src/lib.rs:120.  Infallible by signature: a failure sticks.
    fn copy_page(&mut self, kv: &mut Kv, src: u32, dst: u32) {
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_kv_copy_page(ctx.0, kv.ptr, src, dst) };
    }

    /// crates/yaxus-model/src/lib.rs:123.  The arrays are copied by the library before the
    /// call returns; `pass` may be dropped right after `forward`.
    fn begin_pass(&mut self, pass: &PassMeta) {
        self.rows = pass.pos.len();
        self.ids.clear();
        self.ids.extend_from_slice(&pass.ids);
        let ctx = self.ctx.lock().unwrap();
        unsafe {
            ffi::yx_begin_pass(
                ctx.0,
                pass.pos.len() as u32,
                pass.pos.as_ptr(),
                pass.kv_slot.as_ptr(),
                pass.pt_off.as_ptr(),
                pass.pages.as_ptr(),
                pass.pages.len() as u32,
            )
        };
    }

    /// crates/yaxus-model/src/lib.rs:125.
    fn embed(&mut self, table: &Weight) -> Tensor {
        let (vocab, h) = (table.shape[0], table.shape[1]);
        let out = self.alloc(self.ids.len(), h);
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_embed(ctx.0, table.ptr, vocab as u32, h as u32, self.ids.as_ptr(), self.ids.len() as u32, out.ptr as *mut f32) };
        drop(ctx);
        out
    }

    /// crates/yaxus-model/src/lib.rs:126.
    fn rmsnorm(&mut self, x: &Tensor, w: &Weight, offset: f32, eps: f32) -> Tensor {
        let out = self.alloc(x.rows, x.cols);
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_rmsnorm(ctx.0, x.ptr as *const f32, w.ptr as *const f32, x.rows as u32, x.cols as u32, offset, eps, out.ptr as *mut f32) };
        drop(ctx);
        out
    }

    /// crates/yaxus-model/src/lib.rs:128: `x [T, K] . w[N, K]^T -> [T, N]`.
    fn matmul(&mut self, x: &Tensor, w: &Weight) -> Tensor {
        assert_eq!(x.cols, w.shape[1], "matmul inner dim"); // as the CPU backend asserts (cpu lib.rs:316)
        let out = self.alloc(x.rows, w.shape[0]);
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_matmul(ctx.0, x.ptr as *const f32, w.ptr, x.rows as u32, w.shape[0] as u32, w.shape[1] as u32, out.ptr as *mut f32) };
        drop(ctx);
        out
    }

    /// crates/yaxus-model/src/lib.rs:164-168, one call instead of the default's two.
    fn matmul_glu(&mut self, x: &Tensor, w: &Weight) -> Tensor {
        assert_eq!(x.cols, w.shape[1], "matmul inner dim");
        let out = self.alloc(x.rows, w.shape[0] / 2);
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_matmul_glu(ctx.0, x.ptr as *const f32, w.ptr, x.rows as u32, w.shape[0] as u32, w.shape[1] as u32, out.ptr as *mut f32) };
        drop(ctx);
        out
    }

    /// crates/yaxus-model/src/lib.rs:149-162, one kernel instead of the default's three.
    fn add_norm(&mut self, x: &mut Tensor, delta: &Tensor, post_w: &Weight, post_offset: f32, pre_w: &Weight, pre_offset: f32, eps: f32) -> Tensor {
        let out = self.alloc(x.rows, x.cols);
        let ctx = self.ctx.lock().unwrap();
        unsafe {
            ffi::yx_add_norm(
                ctx.0,
                x.ptr as *mut f32,
                delta.ptr as *const f32,
                post_w.ptr as *const f32,
                post_offset,
                pre_w.ptr as *const f32,
                pre_offset,
                eps,
                x.rows as u32,
                x.cols as u32,
                out.ptr as *mut f32,
            )
        };
        drop(ctx);
        out
    }

    /// crates/yaxus-model/src/lib.rs:132-140: per-head q/k RMSNorm and RoPE, K/V written to each
    /// row's slot, causal (sliding-window where the layer has a window) GQA attention.
    fn attention(&mut self, qkv: &Tensor, q_norm: &Weight, k_norm: &Weight, kv: &mut Kv, cfg: &Config, layer: &LayerMeta) -> Tensor {
        assert_eq!(qkv.rows, self.rows, "attention rows differ from the pass"); // as the CPU backend asserts
        let out = self.alloc(qkv.rows, cfg.num_attention_heads * cfg.head_dim);
        let ctx = self.ctx.lock().unwrap();
        unsafe {
            ffi::yx_attention(
                ctx.0,
                kv.ptr,
                layer.index as i32,
                qkv.ptr as *const f32,
                q_norm.ptr as *const f32,
                k_norm.ptr as *const f32,
                cfg.num_attention_heads as i32,
                cfg.rms_norm_eps,
                out.ptr as *mut f32,
            )
        };
        drop(ctx);
        out
    }

    /// crates/yaxus-model/src/lib.rs:142.
    fn swiglu(&mut self, x: &Tensor) -> Tensor {
        let out = self.alloc(x.rows, x.cols / 2);
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_swiglu(ctx.0, x.ptr as *const f32, x.rows as u32, (x.cols / 2) as u32, out.ptr as *mut f32) };
        drop(ctx);
        out
    }

    /// crates/yaxus-model/src/lib.rs:144.
    fn add_assign(&mut self, a: &mut Tensor, b: &Tensor) {
        assert_eq!(a.rows * a.cols, b.rows * b.cols); // cpu lib.rs:545
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_add_assign(ctx.0, a.ptr as *mut f32, b.ptr as *const f32, a.rows * a.cols) };
    }

    /// crates/yaxus-model/src/lib.rs:170.
    fn select_rows(&mut self, x: &Tensor, rows: &[usize]) -> Tensor {
        let idx: Vec<u32> = rows.iter().map(|&r| r as u32).collect();
        let out = self.alloc(idx.len(), x.cols);
        let ctx = self.ctx.lock().unwrap();
        unsafe { ffi::yx_select_rows(ctx.0, x.ptr as *const f32, x.rows as u32, x.cols as u32, idx.as_ptr(), idx.len() as u32, out.ptr as *mut f32) };
        drop(ctx);
        out
    }
}

impl SyncReadback for CudaBackend {
    /// crates/yaxus-model/src/lib.rs:182.  A read-back: it waits for the device, and a sticky
    /// error is raised to the engine here, as in `to_host`.
    fn argmax_rows(&mut self, logits: &Tensor) -> Vec<u32> {
        let mut v = vec![0u32; logits.rows];
        {
            let ctx = self.ctx.lock().unwrap();
            unsafe { ffi::yx_argmax_rows(ctx.0, logits.ptr as *const f32, logits.rows as u32, logits.cols as u32, v.as_mut_ptr()) };
        }
        if let Err(e) = self.check() {
            panic!("{e:#}");
        }
        v
    }

    /// crates/yaxus-model/src/lib.rs:184.  The trait gives no way to return an error here; like
    /// the reference's GPU backend the failure is raised to the engine, which poisons the step.
    fn to_host(&mut self, x: &Tensor) -> Vec<f32> {
        let mut v = vec![0f32; x.rows * x.cols];
        {
            let ctx = self.ctx.lock().unwrap();
            unsafe { ffi::yx_download(ctx.0, v.as_mut_ptr() as *mut c_void, x.ptr, v.len() * 4, 1) };
        }
        if let Err(e) = self.check() {
            panic!("{e:#}");
        }
        v
    }
}
